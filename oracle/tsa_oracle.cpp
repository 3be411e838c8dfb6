// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of TScale's quantized-attention hot path, used only as the checker in
// tests/, in __graft_entry__.smoke() and as bench.py's CPU baseline.  No product code links,
// imports or calls anything in this file.
//
// Parity pinning: the reference ships no golden vectors for this path, so this restatement is
// pinned against the reference's own CPU code compiled from the reference checkout
// (oracle/_ref/libtsa_ref.so, see oracle/Makefile) - tests/test_oracle_vs_ref.py - and against
// fixtures generated from that library and committed under tests/golden/.
//
// Every function cites the reference code it follows (paths relative to the reference's code/).
// Layouts are dense row-major: vectors [len][H*dim], per-head scalars [H][len].
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <thread>
#include <atomic>
#include <functional>

namespace {

// model_dim.h:19-33: LOG2 = 0.693147f, ATT_DOTPRODUCT_SCALE = 0.5f,
// attDotScale = sqrtf(1/dim) * (0.5f / LOG2)
const float kLog2 = 0.693147f;

inline float AttDotScale(int qDim)
{
    return sqrtf(1.0f / qDim) * (0.5f / kLog2);
}

// heads are independent in every function below: spread them over host threads
// (the reference functions are single-threaded; per-head results do not depend on the split)
int g_threads = 0;

void ParallelFor(int n, const std::function<void(int)> &fn)
{
    int nt = g_threads > 0 ? g_threads : (int)std::thread::hardware_concurrency();
    nt = std::max(1, std::min(nt, n));
    if (nt == 1) {
        for (int i = 0; i < n; ++i) {
            fn(i);
        }
        return;
    }
    std::atomic<int> next(0);
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) {
        pool.emplace_back([&]() {
            for (;;) {
                int i = next.fetch_add(1);
                if (i >= n) {
                    break;
                }
                fn(i);
            }
        });
    }
    for (std::thread &th : pool) {
        th.join();
    }
}

// gpt_cpu.cpp:379-389 CalcDP: sequential fp32 dot, scale, then -slope * (from - to)
inline float CalcDP(const float *qRow, const float *kRow, int qDim, float dotScale, float slope, int from, int to)
{
    float sum = 0;
    for (int x = 0; x < qDim; ++x) {
        sum += qRow[x] * kRow[x];
    }
    float dp = sum * dotScale;
    dp += -(slope) * (from - to);
    return dp;
}

} // namespace

extern "C" {

///////////////////////////////////////////////////////////////////////////////////////////////////
// e4m3 conversions
// decode follows util/fp8.h:4-21 (ConvertE4toFloat); the byte 0x80 decodes to -2^-6 * ... there because
// only x == 0 is special-cased; we keep IEEE-like -0 -> -0.0f (numerically equal to the sum it enters).
float oracle_e4m3_to_f32(int byteVal)
{
    int x = byteVal & 0xff;
    int e = (x >> 3) & 15;
    int m = x & 7;
    float sign = (x & 0x80) ? -1.0f : 1.0f;
    if (e == 0) {
        return sign * ldexpf((float)m, -9);
    }
    return sign * ldexpf(1.0f + m * 0.125f, e - 7);
}

// encode = cvt.rn.satfinite.e4m3x2.f32 (util/fp8.h:48-60 CvtToE4): round to nearest even,
// saturate to +-448, NaN -> 0x7f
int oracle_f32_to_e4m3(float v)
{
    if (std::isnan(v)) {
        return 0x7f;
    }
    int sign = std::signbit(v) ? 0x80 : 0;
    float a = fabsf(v);
    if (a >= 448.0f) {
        return sign | 0x7e;
    }
    if (a < ldexpf(1.0f, -6)) {
        // subnormal: step 2^-9
        float q = nearbyintf(a * 512.0f); // RNE under the default rounding mode
        int m = (int)q;
        return sign | m; // m == 8 gives exponent field 1, mantissa 0 = 2^-6: correct carry
    }
    int ex;
    float fr = frexpf(a, &ex); // a = fr * 2^ex, fr in [0.5, 1)
    int e = ex - 1;            // a = (2 fr) * 2^e
    float mant = nearbyintf((2.0f * fr - 1.0f) * 8.0f);
    int m = (int)mant;
    if (m == 8) {
        m = 0;
        ++e;
    }
    int code = ((e + 7) << 3) | m;
    if (code > 0x7e) {
        code = 0x7e;
    }
    return sign | code;
}

// cvt.rni.sat.s8.f32 (lib/cuda/cuda_util.cuh:33-38) and Float2I8 (gpt_cpu.cpp:15-21): RNE, clamp [-128,127]
int oracle_f32_to_i8(float v)
{
    if (std::isnan(v)) {
        return 0;
    }
    float r = nearbyintf(v);
    if (r > 127.0f) {
        r = 127.0f;
    }
    if (r < -128.0f) {
        r = -128.0f;
    }
    return (int)r;
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// per-row, per-tile quantisers
// kind 0 = RMS (row_tile_scale.cuh:11-34, cuda_matmul.cuh:160-199): scale = sqrt(sum2/tile) * vecScale
// kind 1 = abs-max (row_tile_scale.cuh:59-82, cuda_util.cuh:286-297): scale = max/127 (i8) or max/256 (e4m3)
// kind 2 = RMS with clamp +-127 (cpu_infer.cpp:88-92, 357-391, decode-side NormalizeState)
// dstType 0 = i8, 1 = e4m3.  src [len][xSize] f32, dst [len][xSize] bytes, scale [xSize/tile][len]
void oracle_quant_rows(int kind, int dstType, float vecScale, int len, int xSize, int tile,
    const float *src, int8_t *dst, float *scale)
{
    int tileCount = xSize / tile;
    for (int t = 0; t < len; ++t) {
        for (int tl = 0; tl < tileCount; ++tl) {
            const float *s = src + (size_t)t * xSize + tl * tile;
            int8_t *d = dst + (size_t)t * xSize + tl * tile;
            float discr = 0;
            if (kind == 1) {
                float mx = 0;
                for (int x = 0; x < tile; ++x) {
                    mx = fmaxf(mx, fabsf(s[x]));
                }
                if (mx > 0) {
                    discr = (dstType == 0) ? mx / 127 : mx / 256;
                }
            } else {
                float sum2 = 0;
                for (int x = 0; x < tile; ++x) {
                    sum2 += s[x] * s[x];
                }
                if (sum2 > 0) {
                    discr = sqrtf(sum2 / tile) * vecScale;
                }
            }
            float mult = (discr > 0) ? 1 / discr : 0;
            for (int x = 0; x < tile; ++x) {
                float y = s[x] * mult;
                int q;
                if (dstType == 0) {
                    q = oracle_f32_to_i8(y);
                    if (kind == 2) {
                        q = std::max(-127, std::min(127, q));
                    }
                } else {
                    q = oracle_f32_to_e4m3(y);
                }
                d[x] = (int8_t)q;
            }
            scale[(size_t)tl * len + t] = discr;
        }
    }
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// forward, gpt_cpu.cpp:391-441 (TAttentionComputer::ComputeValLookup)
//   maxDP starts at 0; sumWeight starts at exp2(-maxDP) (the implicit zero vector of weight 1)
// globalScale multiplies attDotScale (gpt_att_fp8.cuh:61 *qvGlobalScale; 1 on the CPU path)
// outputs: out [len][H*vDim]; sumWeight, maxDP, sumWeightLog (= maxDP + log2(sumWeight),
// gpt_att_fp8.cuh:234, gpt_att_fp16.cuh:249) are [H][len]; any of the three may be null
void oracle_att_fwd(int len, int H, int qDim, int vDim, float globalScale, float slope,
    const float *q, const float *k, const float *v, const int *spans, const int *spanPtr,
    float *out, float *sumWeight, float *maxDPArr, float *sumWeightLog)
{
    float dotScale = AttDotScale(qDim) * globalScale;
    size_t qStride = (size_t)H * qDim, vStride = (size_t)H * vDim;
    ParallelFor(H, [&](int head) {
        std::vector<float> acc(vDim);
        for (int from = 0; from < len; ++from) {
            const float *qRow = q + from * qStride + head * qDim;
            float maxDP = 0;
            for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
                for (int to = spans[2 * s]; to <= spans[2 * s + 1]; ++to) {
                    float dp = CalcDP(qRow, k + to * qStride + head * qDim, qDim, dotScale, slope, from, to);
                    maxDP = fmaxf(maxDP, dp);
                }
            }
            float sw = exp2f(-maxDP);
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
                for (int to = spans[2 * s]; to <= spans[2 * s + 1]; ++to) {
                    float dp = CalcDP(qRow, k + to * qStride + head * qDim, qDim, dotScale, slope, from, to);
                    float w = exp2f(dp - maxDP);
                    sw += w;
                    const float *vRow = v + to * vStride + head * vDim;
                    for (int x = 0; x < vDim; ++x) {
                        acc[x] += w * vRow[x];
                    }
                }
            }
            float inv = 1 / sw;
            float *o = out + from * vStride + head * vDim;
            for (int x = 0; x < vDim; ++x) {
                o[x] = acc[x] * inv;
            }
            size_t hi = (size_t)head * len + from;
            if (sumWeight) {
                sumWeight[hi] = sw;
            }
            if (maxDPArr) {
                maxDPArr[hi] = maxDP;
            }
            if (sumWeightLog) {
                sumWeightLog[hi] = maxDP + log2f(sw);
            }
        }
    });
}

// dScale[head][t] = sum_x dOut[t][x] * out[t][x], gpt_cpu.cpp:255-263 (KVProductBackprop tail),
// gpt_att_fp16.cuh:621-643 (CalcDScale)
void oracle_dscale(int len, int H, int vDim, const float *out, const float *dOut, float *dScale)
{
    size_t vStride = (size_t)H * vDim;
    for (int head = 0; head < H; ++head) {
        for (int t = 0; t < len; ++t) {
            dScale[(size_t)head * len + t] = 0;
        }
    }
    for (int t = 0; t < len; ++t) {
        for (int x = 0; x < (int)vStride; ++x) {
            int head = x / vDim;
            dScale[(size_t)head * len + t] += dOut[t * vStride + x] * out[t * vStride + x];
        }
    }
}

// backward, gpt_cpu.cpp:465-555 (CalcDDot, GradQK, GradQV)
//   w = exp2(dp - maxDP) / sumWeight;  dW = sum_x dOut[from][x] * v[to][x]
//   dDot = w * (dW - dScale[head][from]) * attDotScale * LOG2
//   dq[from] += dDot * k[to];  dk[to] += dDot * q[from];  dv[to] += w * dOut[from]
// dq is accumulated in span order per row (GradQK); dk/dv in transposed-span order per key (GradQV)
void oracle_att_bwd(int len, int H, int qDim, int vDim, float globalScale, float slope,
    const float *q, const float *k, const float *v, const float *dOut, const float *dScale,
    const float *sumWeight, const float *maxDPArr,
    const int *spans, const int *spanPtr, const int *revSpans, const int *revSpanPtr,
    float *dq, float *dk, float *dv)
{
    float dotScale = AttDotScale(qDim) * globalScale;
    size_t qStride = (size_t)H * qDim, vStride = (size_t)H * vDim;
    memset(dq, 0, sizeof(float) * len * qStride);
    memset(dk, 0, sizeof(float) * len * qStride);
    memset(dv, 0, sizeof(float) * len * vStride);
    ParallelFor(H, [&](int head) {
        auto dDotFn = [&](int from, int to, float dp, float *pW) {
            size_t hi = (size_t)head * len + from;
            float w = exp2f(dp - maxDPArr[hi]) / sumWeight[hi];
            float dW = 0;
            const float *doRow = dOut + from * vStride + head * vDim;
            const float *vRow = v + to * vStride + head * vDim;
            for (int x = 0; x < vDim; ++x) {
                dW += doRow[x] * vRow[x];
            }
            *pW = w;
            return w * (dW - dScale[hi]) * dotScale * kLog2;
        };
        for (int from = 0; from < len; ++from) {
            const float *qRow = q + from * qStride + head * qDim;
            float *dqRow = dq + from * qStride + head * qDim;
            for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
                for (int to = spans[2 * s]; to <= spans[2 * s + 1]; ++to) {
                    const float *kRow = k + to * qStride + head * qDim;
                    float dp = CalcDP(qRow, kRow, qDim, dotScale, slope, from, to);
                    float w;
                    float dDot = dDotFn(from, to, dp, &w);
                    for (int x = 0; x < qDim; ++x) {
                        dqRow[x] += dDot * kRow[x];
                    }
                }
            }
        }
        for (int to = 0; to < len; ++to) {
            const float *kRow = k + to * qStride + head * qDim;
            float *dkRow = dk + to * qStride + head * qDim;
            float *dvRow = dv + to * vStride + head * vDim;
            for (int s = revSpanPtr[to]; s < revSpanPtr[to + 1]; ++s) {
                for (int from = revSpans[2 * s]; from <= revSpans[2 * s + 1]; ++from) {
                    const float *qRow = q + from * qStride + head * qDim;
                    float dp = CalcDP(qRow, kRow, qDim, dotScale, slope, from, to);
                    float w;
                    float dDot = dDotFn(from, to, dp, &w);
                    for (int x = 0; x < qDim; ++x) {
                        dkRow[x] += dDot * qRow[x];
                    }
                    const float *doRow = dOut + from * vStride + head * vDim;
                    for (int x = 0; x < vDim; ++x) {
                        dvRow[x] += w * doRow[x];
                    }
                }
            }
        }
    });
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// exact integer scores: S[head][from][to] = sum_x q8[from][x] * k8[to][x]
// (cpu_infer.cpp:199-210 DotInt8; GPU twin gpt_att_fp16.cuh:76-101 s8 -> s32 tiles)
void oracle_qk_int32(int lenQ, int lenK, int H, int qDim, const int8_t *q8, const int8_t *k8, int32_t *S)
{
    size_t stride = (size_t)H * qDim;
    ParallelFor(H, [&](int head) {
        for (int from = 0; from < lenQ; ++from) {
            const int8_t *a = q8 + from * stride + head * qDim;
            for (int to = 0; to < lenK; ++to) {
                const int8_t *b = k8 + to * stride + head * qDim;
                int32_t sum = 0;
                for (int x = 0; x < qDim; ++x) {
                    sum += (int32_t)a[x] * (int32_t)b[x];
                }
                S[((size_t)head * lenQ + from) * lenK + to] = sum;
            }
        }
    });
}

void oracle_set_threads(int n)
{
    g_threads = n;
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// decode step, cpu_infer.cpp:413-460 (NCPUInfer::ComputeValLookup) for one sequence.
// Cache holds ctxLen tokens including the one just appended; cur = ctxLen - 1.
// Keys: width == 0 -> {cur}; else to = cur - dt, dt = 1..min(cur, width)   (:421-431)
// logit = int32dot * kScale[to][h] * (attDotScale * qScale[h]) - slope * (cur - to), sink logit 0 first (:444-449)
// out   = sum softmax * vScale * v8[to]                                              (:452-458)
// The reference has constant query and value scales (VEC_SCALE = 1/24); here they are per head
// (qScale [H]) and per (token, head) (vScale [ctxLen][H]) so that constants reproduce it.
// expMode 0: the reference's AVX2 polynomial 2^x (TSoftMaxBuf::SoftMax :243-281), fp32, evaluated
//            with fused multiply-adds like _mm256_fmadd_ps; expMode 1: exact exp2f.
static float RefPolyExp2(float xIn)
{
    float x = fmaxf(xIn, -127.0f);
    float xf = floorf(x);
    x = x - xf;
    int xfi = (int)nearbyintf(xf);
    float x2 = x * x;
    const float c0 = -3.069678791803394491901405992213472390777e-1f;
    const float c1 = -6.558811624324781017147952441210509604385e-2f;
    const float c2 = -1.355574723481491770403079319055785445381e-2f;
    float res = fmaf(fmaf(c2, x, c1), x, c0);
    float xBy1mx = x - x2;
    res = fmaf(res, xBy1mx, x);
    res = res + 1.0f;
    int32_t bits;
    memcpy(&bits, &res, 4);
    bits += xfi << 23;
    memcpy(&res, &bits, 4);
    return res;
}

void oracle_decode_step(int ctxLen, int H, int D, int width, float slope, int expMode,
    const int8_t *kCache, const float *kScale, const int8_t *vCache, const float *vScale,
    const int8_t *q8, const float *qScale, float *out)
{
    int cur = ctxLen - 1;
    std::vector<int> toArr;
    if (width == 0) {
        toArr.push_back(cur);
    } else {
        int ww = std::min(cur, width);
        for (int dt = 1; dt <= ww; ++dt) {
            toArr.push_back(cur - dt);
        }
    }
    int toCount = (int)toArr.size();
    size_t stride = (size_t)H * D;
    float attDotScale = AttDotScale(D);
    for (int i = 0; i < (int)stride; ++i) {
        out[i] = 0;
    }
    // the reference evaluates 8 lanes at a time and sums lanes; lane order matters for bit parity
    for (int head = 0; head < H; ++head) {
        std::vector<float> buf;
        buf.push_back(0.0f);
        float maxValue = 0;
        for (int z = 0; z < toCount; ++z) {
            int to = toArr[z];
            const int8_t *a = q8 + head * D;
            const int8_t *b = kCache + to * stride + head * D;
            int32_t dot = 0;
            for (int x = 0; x < D; ++x) {
                dot += (int32_t)a[x] * (int32_t)b[x];
            }
            float logit = dot * kScale[(size_t)to * H + head] * attDotScale * qScale[head] - slope * (cur - to);
            buf.push_back(logit);
            maxValue = std::max(maxValue, logit);
        }
        int n = (int)buf.size();
        int padded = (n + 7) / 8 * 8;
        buf.resize(padded, -1e38f);
        float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < padded; ++i) {
            float e = (expMode == 0) ? RefPolyExp2(buf[i] - maxValue) : exp2f(fmaxf(buf[i] - maxValue, -127.0f));
            buf[i] = e;
            lanes[i & 7] += e;
        }
        // HorizontalSum (gpt/model_params/sse_utils.h:208-228): ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7))
        float total = ((lanes[0] + lanes[4]) + (lanes[2] + lanes[6])) + ((lanes[1] + lanes[5]) + (lanes[3] + lanes[7]));
        float scale = 1 / total;
        float *o = out + head * D;
        for (int z = 0; z < toCount; ++z) {
            int to = toArr[z];
            float w = buf[z + 1] * scale * vScale[(size_t)to * H + head];
            const int8_t *vr = vCache + to * stride + head * D;
            for (int x = 0; x < D; ++x) {
                o[x] += w * vr[x];
            }
        }
    }
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// span preprocessing
// TransposeAttention, att/att.cpp:26-56: for every (from, to) pair in row order, extend the last
// span of `to` if it ends at from-1, else open a new one.  Returns span count (or -needed).
int oracle_transpose_attention(int len, const int *spans, const int *spanPtr, int maxSpans, int *resSpans, int *resSpanPtr)
{
    std::vector<std::vector<int>> rows(len);
    for (int from = 0; from < len; ++from) {
        for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
            for (int to = spans[2 * s]; to <= spans[2 * s + 1]; ++to) {
                std::vector<int> &dst = rows[to];
                if (!dst.empty() && dst.back() == from - 1) {
                    dst.back() = from;
                } else {
                    dst.push_back(from);
                    dst.push_back(from);
                }
            }
        }
    }
    int total = 0;
    for (int t = 0; t < len; ++t) {
        total += (int)rows[t].size() / 2;
    }
    if (total > maxSpans) {
        return -total;
    }
    int ptr = 0;
    resSpanPtr[0] = 0;
    for (int t = 0; t < len; ++t) {
        for (size_t i = 0; i < rows[t].size(); ++i) {
            resSpans[ptr * 2 + (int)i] = rows[t][i];
        }
        ptr += (int)rows[t].size() / 2;
        resSpanPtr[t + 1] = ptr;
    }
    return total;
}

// GroupAttention<64,128>, att/att.h:95-181.  Spans of each row are sorted by start; round r of a
// 64-row block takes the r-th remaining span of every row that still has one (the reference's
// take-condition `a >= start/ALIGN || ...` is always true because start is the minimum), so a group
// holds at most one span per row.  Start/Finish are the min start / max finish rounded down to 128.
// Record = {Start, Finish, SpanStart[64], SpanFinish[64]}; unused rows hold (1e9, 1e9-1).
int oracle_group_attention_64_128(int len, const int *spans, const int *spanPtr, int maxGroups, int *groups, int *groupPtr)
{
    const int N = 64, ALIGN = 128, FAR_RIGHT = 1000000000;
    int blockCount = (len + N - 1) / N;
    int total = 0;
    groupPtr[0] = 0;
    for (int pass = 0; pass < 2; ++pass) {
        total = 0;
        for (int g = 0; g < blockCount; ++g) {
            std::vector<std::vector<std::pair<int, int>>> rowSpans(N);
            size_t rounds = 0;
            for (int kk = 0; kk < N; ++kk) {
                int from = g * N + kk;
                if (from < len) {
                    for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
                        rowSpans[kk].push_back({spans[2 * s], spans[2 * s + 1]});
                    }
                    std::stable_sort(rowSpans[kk].begin(), rowSpans[kk].end(),
                        [](const std::pair<int, int> &a, const std::pair<int, int> &b) { return a.first < b.first; });
                    rounds = std::max(rounds, rowSpans[kk].size());
                }
            }
            for (size_t r = 0; r < rounds; ++r) {
                if (pass == 1) {
                    int *rec = groups + (size_t)total * 130;
                    int gStart = FAR_RIGHT, gFinish = 0;
                    for (int kk = 0; kk < N; ++kk) {
                        if (r < rowSpans[kk].size()) {
                            rec[2 + kk] = rowSpans[kk][r].first;
                            rec[2 + N + kk] = rowSpans[kk][r].second;
                            gStart = std::min(gStart, rowSpans[kk][r].first);
                            gFinish = std::max(gFinish, rowSpans[kk][r].second);
                        } else {
                            rec[2 + kk] = FAR_RIGHT;
                            rec[2 + N + kk] = FAR_RIGHT - 1;
                        }
                    }
                    rec[0] = gStart / ALIGN * ALIGN;
                    rec[1] = gFinish / ALIGN * ALIGN;
                }
                ++total;
            }
            if (pass == 1) {
                groupPtr[g + 1] = total;
            }
        }
        if (pass == 0 && total > maxGroups) {
            return -total;
        }
    }
    return total;
}

}

///////////////////////////////////////////////////////////////////////////////////////////////////
// producer of the attention inputs: per-head RMS normalise, rope, quantise
// FillRopeBuf (code/gpt/att/rope.cpp:4-24): theta = 500000; per 64-element block the first 32 entries hold cos, the
// next 32 sin of angle t * theta^(-(2k)/width), k = block/2 + index
extern "C" void oracle_fill_rope(int width, int maxLen, float *rope)
{
    float theta = 500000;
    std::vector<float> freq;
    for (int k = 0; k < width / 2; ++k) {
        freq.push_back((float)exp(-logf(theta) * (k * 2. / width))); // float log, double product and exp, as the reference's overloads resolve
    }
    for (int t = 0; t < maxLen; ++t) {
        for (int base = 0; base < width; base += 64) {
            for (int k = 0; k < 32; ++k) {
                float angle = t * freq[base / 2 + k];
                rope[(size_t)t * width + base + k] = cosf(angle);
                rope[(size_t)t * width + base + k + 32] = sinf(angle);
            }
        }
    }
}

// ReferenceApplyRope (rope.cpp:28-46): inside every head, elements k and k + 32 of a 64-element block rotate by the
// block's angle; dir = -1 rotates back.  data [len][dim] in place, rope [len][headDim]
extern "C" void oracle_apply_rope(int headDim, int len, int dim, float dir, const float *rope, float *data)
{
    for (int t = 0; t < len; ++t) {
        float *row = data + (size_t)t * dim;
        const float *rp = rope + (size_t)t * headDim;
        for (int offset = 0; offset < dim; offset += headDim) {
            for (int blk = 0; blk < headDim; blk += 64) {
                for (int k = 0; k < 32; ++k) {
                    float v0 = row[offset + blk + k], v1 = row[offset + blk + k + 32];
                    float cosValue = rp[blk + k];
                    float sinValue = rp[blk + k + 32] * dir;
                    row[offset + blk + k] = v0 * cosValue - v1 * sinValue;
                    row[offset + blk + k + 32] = v0 * sinValue + v1 * cosValue;
                }
            }
        }
    }
}

// normalise (row_tile_scale.cuh:11-34 / cuda_matmul.cuh:147-204: discr = sqrt(sum2 / D) * vecScale, x / discr), rope
// (gpt_rope.cuh:37-51 applies it to the normalised vector), quantise; roped [len][dim] (may be null) receives the
// fp32 vectors before quantisation.  dstType 0 = i8, 1 = e4m3; scale [dim/headDim][len]
extern "C" void oracle_norm_rope_quant(int dstType, float vecScale, int len, int dim, int headDim, float dir,
    const float *src, const float *rope, int8_t *dst, float *scale, float *roped)
{
    int heads = dim / headDim;
    std::vector<float> rowBuf(dim);
    for (int t = 0; t < len; ++t) {
        for (int h = 0; h < heads; ++h) {
            const float *s = src + (size_t)t * dim + h * headDim;
            float sum2 = 0;
            for (int x = 0; x < headDim; ++x) {
                sum2 += s[x] * s[x];
            }
            float discr = 0;
            if (sum2 > 0) {
                discr = sqrtf(sum2 / headDim) * vecScale;
            }
            float mult = (discr > 0) ? 1 / discr : 0;
            for (int x = 0; x < headDim; ++x) {
                rowBuf[h * headDim + x] = s[x] * mult;
            }
            scale[(size_t)h * len + t] = discr;
        }
        if (rope) {
            oracle_apply_rope(headDim, 1, dim, dir, rope + (size_t)t * headDim, rowBuf.data());
        }
        for (int x = 0; x < dim; ++x) {
            float y = rowBuf[x];
            if (roped) {
                roped[(size_t)t * dim + x] = y;
            }
            dst[(size_t)t * dim + x] = (int8_t)(dstType == 0 ? oracle_f32_to_i8(y) : oracle_f32_to_e4m3(y));
        }
    }
}

// back-propagation through the producer's fp32 stage: inverse rope (ApplyRope with the opposite direction, gpt_cpu.cpp:
// 759-760), then NormalizeStateBackward (gpt_cpu.cpp:329-360): grad = sqrt(D / sum2) * (g - src * dot(src, g) / sum2).
// src: raw projections [len][dim]; dRoped: gradient with respect to the roped unit-RMS vectors; rope may be null
extern "C" void oracle_rope_norm_bwd(int len, int dim, int headDim, float dir, const float *src, const float *dRoped,
    const float *rope, float *grad)
{
    std::vector<float> g(dim);
    for (int t = 0; t < len; ++t) {
        for (int x = 0; x < dim; ++x) {
            g[x] = dRoped[(size_t)t * dim + x];
        }
        if (rope) {
            oracle_apply_rope(headDim, 1, dim, -dir, rope + (size_t)t * headDim, g.data());
        }
        for (int offset = 0; offset < dim; offset += headDim) {
            const float *sp = src + (size_t)t * dim + offset;
            float sum2 = 0, dp = 0;
            for (int x = 0; x < headDim; ++x) {
                sum2 += sp[x] * sp[x];
                dp += sp[x] * g[offset + x];
            }
            float *dst = grad + (size_t)t * dim + offset;
            if (sum2 == 0) {
                for (int x = 0; x < headDim; ++x) {
                    dst[x] = 0;
                }
            } else {
                float sigma = dp / sum2;
                float scale = sqrtf(headDim / sum2);
                for (int x = 0; x < headDim; ++x) {
                    dst[x] = scale * (g[offset + x] - sp[x] * sigma);
                }
            }
        }
    }
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// consumer of the attention output: the combiner input (gpt_cpu.cpp:191-216) and its back-propagation (219-262).
// kv[t][head * D * 4 + blk * D + z] = k[t][head * D + (z ^ blk)] * val[t][head * D + z],  blk = 0 .. 3 (COMBINER_REP)
extern "C" void oracle_kv_product(int len, int H, int D, const float *k, const float *val, float *kv)
{
    const int REP = 4;
    for (int t = 0; t < len; ++t) {
        for (int head = 0; head < H; ++head) {
            const float *kp = k + ((size_t)t * H + head) * D;
            const float *vp = val + ((size_t)t * H + head) * D;
            for (int blk = 0; blk < REP; ++blk) {
                float *dst = kv + (size_t)t * H * D * REP + (size_t)head * D * REP + blk * D;
                for (int z = 0; z < D; ++z) {
                    dst[z] = kp[z ^ blk] * vp[z];
                }
            }
        }
    }
}

// dK[z] = sum_blk dkv[blk][z ^ blk] * val[z ^ blk];  dVal[z] = sum_blk dkv[blk][z] * k[z ^ blk];  dScale[head][t] =
// sum_z dVal[z] * val[z] (the quantity the attention backward calls dScale)
extern "C" void oracle_kv_product_bwd(int len, int H, int D, const float *k, const float *val, const float *dkv,
    float *dK, float *dVal, float *dScale)
{
    const int REP = 4;
    for (int t = 0; t < len; ++t) {
        for (int head = 0; head < H; ++head) {
            const float *kp = k + ((size_t)t * H + head) * D;
            const float *vp = val + ((size_t)t * H + head) * D;
            float *dk = dK + ((size_t)t * H + head) * D;
            float *dv = dVal + ((size_t)t * H + head) * D;
            for (int z = 0; z < D; ++z) {
                dk[z] = 0;
                dv[z] = 0;
            }
            for (int blk = 0; blk < REP; ++blk) {
                const float *g = dkv + (size_t)t * H * D * REP + (size_t)head * D * REP + blk * D;
                for (int z = 0; z < D; ++z) {
                    dk[z] += g[z ^ blk] * vp[z ^ blk];
                    dv[z] += g[z] * kp[z ^ blk];
                }
            }
            float sum = 0;
            for (int z = 0; z < D; ++z) {
                sum += dv[z] * vp[z];
            }
            dScale[(size_t)head * len + t] = sum;
        }
    }
}

///////////////////////////////////////////////////////////////////////////////////////////////////
// one-token inference step through the int8 model with per-layer KV caches
// (NCPUInfer::ComputePrediction / AddLookupProduct, code/gpt/train/cpu_infer.cpp:466-560).
// Matrices are row-major int8 [rows][cols]; same argument layout as ref_infer_create of the reference shim.
namespace {
const float kVecScale = 1.0f / 24; // VEC_SCALE, cpu_infer.cpp:16

struct TInferLayer
{
    const int8_t *QK, *QV, *K, *V, *Combiner, *Expand, *Contract;
    float QVScale, CombinerScale, ContractScale, Slope;
    int Width;
    std::vector<int8_t> KeyCache, ValCache; // [t][H*D]
    std::vector<float> KeyScale, ValScale;  // [t][H]
};

struct TInferOracle
{
    int Dim, HeadDim, HeadCount, ReluDim, Vocab, LabelCount, RopeLen, T = 0, ExpMode = 1;
    std::vector<TInferLayer> Layers;
    const int8_t *LabelEmbed, *FinalLayer;
    float LabelEmbedScale, FinalLayerScale;
    const float *Bias;
    std::vector<float> Rope;
    std::vector<float> Logits;
};

// ConvertToInt8 (cpu_infer.cpp:88-92): round to nearest even, clamp to +-127
int8_t InferToInt8(float x)
{
    float r = nearbyintf(x);
    r = r > 127.0f ? 127.0f : (r < -127.0f ? -127.0f : r);
    return (int8_t)r;
}

// NormalizeState (cpu_infer.cpp:357-391): groups of dim / groups elements, sequential float sum of squares
void InferNormalize(const float *src, int dim, int groups, int8_t *dst, float *groupScale)
{
    int gd = dim / groups;
    for (int h = 0; h < groups; ++h) {
        const float *s = src + h * gd;
        float sum2 = 0;
        for (int x = 0; x < gd; ++x) {
            sum2 += s[x] * s[x];
        }
        if (sum2 == 0) {
            for (int x = 0; x < gd; ++x) {
                dst[h * gd + x] = 0;
            }
            if (groupScale) {
                groupScale[h] = 0;
            }
        } else {
            float sko = sqrtf(sum2 / gd);
            float discrScale = sko * kVecScale;
            float mult = 1 / discrScale;
            for (int x = 0; x < gd; ++x) {
                dst[h * gd + x] = InferToInt8(s[x] * mult);
            }
            if (groupScale) {
                groupScale[h] = discrScale;
            }
        }
    }
}

// MulForward (cpu_infer.cpp:282-293): exact int32 dot products of the vector with every matrix row, as floats
void InferMul(const int8_t *vec, const int8_t *mat, int rows, int cols, float *res)
{
    for (int k = 0; k < rows; ++k) {
        int32_t dot = 0;
        for (int x = 0; x < cols; ++x) {
            dot += (int32_t)vec[x] * (int32_t)mat[(size_t)k * cols + x];
        }
        res[k] = (float)dot;
    }
}
} // namespace

extern "C" void *oracle_infer_create(int dim, int headDim, int headCount, int reluMult, int vocab, int labelCount, int layerCount, int ropeLen,
    const int8_t *const *layerMats, const float *layerScalars, const int8_t *labelEmbed, float labelEmbedScale,
    const int8_t *finalLayer, float finalLayerScale, const float *bias)
{
    TInferOracle *h = new TInferOracle;
    h->Dim = dim;
    h->HeadDim = headDim;
    h->HeadCount = headCount;
    h->ReluDim = headCount * 128 * reluMult; // TModelDims::GetReluDim, model_dim.h:66
    h->Vocab = vocab;
    h->LabelCount = labelCount;
    h->RopeLen = ropeLen;
    h->Layers.resize(layerCount);
    for (int d = 0; d < layerCount; ++d) {
        TInferLayer &l = h->Layers[d];
        const int8_t *const *m = layerMats + d * 7;
        l.QK = m[0], l.QV = m[1], l.K = m[2], l.V = m[3], l.Combiner = m[4], l.Expand = m[5], l.Contract = m[6];
        const float *s = layerScalars + d * 5;
        l.QVScale = s[0], l.CombinerScale = s[1], l.ContractScale = s[2], l.Width = (int)s[3], l.Slope = s[4];
    }
    h->LabelEmbed = labelEmbed;
    h->LabelEmbedScale = labelEmbedScale;
    h->FinalLayer = finalLayer;
    h->FinalLayerScale = finalLayerScale;
    h->Bias = bias;
    h->Rope.resize((size_t)ropeLen * headDim);
    oracle_fill_rope(headDim, ropeLen, h->Rope.data());
    return h;
}

// expMode 0: the reference's polynomial 2^x, 1: exact exp2f
extern "C" void oracle_infer_set_exp(void *handle, int expMode)
{
    ((TInferOracle *)handle)->ExpMode = expMode;
}

// prediction [vocab] (may be null); logits [vocab] (may be null) receives the int32 products of the final layer as floats
extern "C" void oracle_infer_step(void *handle, const int *labels, int labelCount, float *prediction, float *logits)
{
    TInferOracle &m = *(TInferOracle *)handle;
    const int dim = m.Dim, H = m.HeadCount, D = m.HeadDim, hs = H * D, reluDim = m.ReluDim;
    std::vector<float> state(dim, 0.0f);
    for (int i = 0; i < labelCount; ++i) {
        for (int x = 0; x < dim; ++x) {
            state[x] += m.LabelEmbed[(size_t)labels[i] * dim + x] * m.LabelEmbedScale;
        }
    }
    std::vector<int8_t> norm(std::max(dim, reluDim)), qk(hs), qv(hs), k(hs), v(hs), kv((size_t)hs * 4), relu(reluDim);
    std::vector<float> qkSrc(hs), qvSrc(hs), kSrc(hs), vSrc(hs), qvScale(H), vScale(H, kVecScale), qScale(H, kVecScale), val(hs), delta(dim),
        reluSrc(reluDim);
    const float *rope = m.Rope.data() + (size_t)m.T * D;
    for (TInferLayer &l : m.Layers) {
        InferNormalize(state.data(), dim, dim / 128, norm.data(), nullptr); // STATE_NORM_TILE = 128
        InferMul(norm.data(), l.QK, hs, dim, qkSrc.data());
        InferMul(norm.data(), l.QV, hs, dim, qvSrc.data());
        InferMul(norm.data(), l.K, hs, dim, kSrc.data());
        InferMul(norm.data(), l.V, hs, dim, vSrc.data());
        oracle_apply_rope(D, 1, hs, 1.0f, rope, qkSrc.data());
        oracle_apply_rope(D, 1, hs, 1.0f, rope, qvSrc.data());
        InferNormalize(qkSrc.data(), hs, H, qk.data(), nullptr);
        InferNormalize(qvSrc.data(), hs, H, qv.data(), qvScale.data());
        InferNormalize(kSrc.data(), hs, H, k.data(), nullptr);
        InferNormalize(vSrc.data(), hs, H, v.data(), nullptr);
        const float qvMult = l.QVScale * kVecScale * sqrtf(1.0f / dim);
        for (float &x : qvScale) {
            x *= qvMult;
        }
        l.KeyCache.insert(l.KeyCache.end(), qv.begin(), qv.end());
        l.ValCache.insert(l.ValCache.end(), v.begin(), v.end());
        l.KeyScale.insert(l.KeyScale.end(), qvScale.begin(), qvScale.end());
        l.ValScale.insert(l.ValScale.end(), vScale.begin(), vScale.end());
        int ctxLen = (int)(l.KeyCache.size() / hs);
        oracle_decode_step(ctxLen, H, D, l.Width, l.Slope, m.ExpMode, l.KeyCache.data(), l.KeyScale.data(), l.ValCache.data(), l.ValScale.data(),
            qk.data(), qScale.data(), val.data());
        // KVProduct (cpu_infer.cpp:318-337)
        for (int head = 0; head < H; ++head) {
            for (int blk = 0; blk < 4; ++blk) {
                for (int z = 0; z < D; ++z) {
                    kv[(size_t)head * D * 4 + blk * D + z] = InferToInt8(k[head * D + (z ^ blk)] * val[head * D + z]);
                }
            }
        }
        InferMul(kv.data(), l.Combiner, dim, hs * 4, delta.data());
        const float combScale = l.CombinerScale * kVecScale * sqrtf(1.0f / (hs * 4));
        for (int x = 0; x < dim; ++x) {
            state[x] += delta[x] * combScale;
        }
        InferNormalize(state.data(), dim, dim / 128, norm.data(), nullptr);
        InferMul(norm.data(), l.Expand, reluDim, dim, reluSrc.data());
        InferNormalize(reluSrc.data(), reluDim, H, relu.data(), nullptr);
        for (int8_t &x : relu) {
            x = std::max<int8_t>(0, x);
        }
        InferMul(relu.data(), l.Contract, dim, reluDim, delta.data());
        const float contractScale = l.ContractScale * kVecScale * sqrtf(1.0f / reluDim);
        for (int x = 0; x < dim; ++x) {
            state[x] += delta[x] * contractScale;
        }
    }
    if (prediction || logits) {
        InferNormalize(state.data(), dim, dim / 128, norm.data(), nullptr);
        m.Logits.resize(m.Vocab);
        InferMul(norm.data(), m.FinalLayer, m.Vocab, dim, m.Logits.data());
        if (logits) {
            memcpy(logits, m.Logits.data(), sizeof(float) * m.Vocab);
        }
        if (prediction) {
            // SoftMax (cpu_infer.cpp:340-354) over TSoftMaxBuf (cpu_infer.cpp:216-268): the maximum starts at 0
            const float finalScale = sqrtf(1.0f / dim) * (1.0f / 0.693147f) * m.FinalLayerScale * kVecScale;
            int padded = (m.Vocab + 7) / 8 * 8;
            std::vector<float> buf(std::max(padded, 8), -1e38f);
            float maxValue = 0;
            for (int x = 0; x < m.Vocab; ++x) {
                buf[x] = m.Logits[x] * finalScale + m.Bias[x];
                maxValue = std::max(maxValue, buf[x]);
            }
            float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int i = 0; i < padded; ++i) {
                float e = (m.ExpMode == 0) ? RefPolyExp2(buf[i] - maxValue) : exp2f(fmaxf(buf[i] - maxValue, -127.0f));
                buf[i] = e;
                lanes[i & 7] += e;
            }
            float total = ((lanes[0] + lanes[4]) + (lanes[2] + lanes[6])) + ((lanes[1] + lanes[5]) + (lanes[3] + lanes[7]));
            float scale = 1 / total;
            for (int x = 0; x < m.Vocab; ++x) {
                prediction[x] = buf[x] * scale;
            }
        }
    }
    m.T += 1;
}

extern "C" void oracle_infer_free(void *handle)
{
    delete (TInferOracle *)handle;
}
