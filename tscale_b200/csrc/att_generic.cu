// SIMT attention kernels that accept every mask and head size the ABI allows: the path taken for
// multi-round span lists, odd head sizes and int8 values, and the backward.
//
// Math (reference: TAttentionComputer, code/gpt/compute/gpt_cpu.cpp:379-555; GPU twins
// gpt_att_fp16.cuh:121-318, 332-616):
//   z_ij = dot(q8_i, k8_j) * sq_i * sk_j * c - slope * (i - j),  c = sqrt(1/Dq) * 0.5/LOG2 * g
//   m_i = max(0, max_j z_ij);  Z_i = 2^-m_i + sum_j 2^(z_ij - m_i);  O_i = sum_j 2^(z_ij - m_i) sv_j v8_j / Z_i
//   lse_i = m_i + log2 Z_i
//   p_ij = 2^(z_ij - lse_i); dP_ij = dO_i . (sv_j v8_j); dS_ij = p_ij (dP_ij - delta_i) c ln2
//   dq_i = sum_j dS_ij sk_j k8_j;  dk_j = sum_i dS_ij sq_i q8_i;  dv_j = sum_i p_ij dO_i
// One warp owns one (row, head).  Lanes take one key (or query) each for the dot products; the
// weighted sums are formed by broadcasting each lane's weight and reading the 8-bit rows coalesced.
// Integer dots are exact: 8-bit values are summed in fp32 below 2^24.
#include "att_internal.cuh"

namespace tsa {

__device__ __forceinline__ float RowDot(const float *a, const uint8_t *row, int dim, int dt)
{
    // a: smem vector (broadcast reads), row: this lane's 8-bit row, 4 bytes per load
    float sum = 0;
    const uint32_t *r4 = reinterpret_cast<const uint32_t *>(row);
    if (dt == TSA_I8) {
        for (int x = 0; x < dim; x += 4) {
            uint32_t w = r4[x >> 2];
            sum += a[x] * (float)(int8_t)(w) + a[x + 1] * (float)(int8_t)(w >> 8) + a[x + 2] * (float)(int8_t)(w >> 16) + a[x + 3] * (float)(int8_t)(w >> 24);
        }
    } else {
        for (int x = 0; x < dim; x += 4) {
            uint32_t w = r4[x >> 2];
            float2 lo = UnpackE4M3x2(w & 0xffff), hi = UnpackE4M3x2(w >> 16);
            sum += a[x] * lo.x + a[x + 1] * lo.y + a[x + 2] * hi.x + a[x + 3] * hi.y;
        }
    }
    return sum;
}

__device__ __forceinline__ float RowDotF(const float *a, const void *row, int base, int dim, int dt)
{
    float sum = 0;
    for (int x = 0; x < dim; ++x) {
        sum += a[x] * LoadAsFloat(row, base + x, dt);
    }
    return sum;
}

__device__ __forceinline__ float Load8(const uint8_t *row, int idx, int dt)
{
    return dt == TSA_I8 ? (float)(int8_t)row[idx] : E4M3ToFloat(row[idx]);
}

// ---- forward --------------------------------------------------------------------------------
__global__ void __launch_bounds__(GEN_WARPS * 32) GenericFwdKernel(TGenParams p)
{
    __shared__ float qs[GEN_WARPS][GEN_MAX_DIM];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int i = blockIdx.x * GEN_WARPS + warp;
    int head = blockIdx.y;
    if (i >= p.Len) {
        return;
    }
    float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
    float c = p.C * g;
    const uint8_t *qRow = p.Q.Row(i) + head * p.Dq;
    for (int x = lane; x < p.Dq; x += 32) {
        qs[warp][x] = Load8(qRow, x, p.QkDtype);
    }
    __syncwarp();
    float sq = p.QScale.Valid() ? p.QScale.Row(head)[i] : p.QkVecScale;
    float rowMult = sq * c;
    float m = 0, l = 0;
    float acc[GEN_ACC];
#pragma unroll
    for (int t = 0; t < GEN_ACC; ++t) {
        acc[t] = 0;
    }
    int blk = i / TSA_ATT_GROUP, r = i % TSA_ATT_GROUP;
    for (int gi = p.SpanPtr[blk]; gi < p.SpanPtr[blk + 1]; ++gi) {
        int s = max(p.Spans[gi].SpanStart[r], 0), f = min(p.Spans[gi].SpanFinish[r], p.KeyRows - 1);
        for (int j0 = s; j0 <= f; j0 += 32) {
            int j = j0 + lane;
            bool ok = j <= f;
            float z = -1e30f, sv = 0;
            if (ok) {
                float dot = RowDot(qs[warp], p.K.Row(j) + head * p.Dq, p.Dq, p.QkDtype);
                z = dot * p.KScale.Row(head)[j] * rowMult - p.Slope * (float)(i - j);
                sv = p.VScale.Valid() ? p.VScale.Row(head)[j] : p.VVecScale;
            }
            float nm = fmaxf(m, WarpMax(z));
            float corr = exp2f(m - nm);
            m = nm;
            l *= corr;
#pragma unroll
            for (int t = 0; t < GEN_ACC; ++t) {
                acc[t] *= corr;
            }
            float w = ok ? exp2f(z - m) : 0.0f;
            l += w;
            float wv = w * sv;
            int cnt = min(32, f - j0 + 1);
            for (int jj = 0; jj < cnt; ++jj) {
                float wj = __shfl_sync(0xffffffffu, wv, jj);
                const uint8_t *vRow = p.V.Row(j0 + jj) + head * p.Dv;
#pragma unroll
                for (int t = 0; t < GEN_ACC; ++t) {
                    int x = lane + 32 * t;
                    if (x < p.Dv) {
                        acc[t] += wj * Load8(vRow, x, p.VDtype);
                    }
                }
            }
        }
    }
    l = WarpSum(l) + exp2f(-m);
    float inv = 1.0f / l;
    void *oRow = p.Out.Row(i);
#pragma unroll
    for (int t = 0; t < GEN_ACC; ++t) {
        int x = lane + 32 * t;
        if (x < p.Dv) {
            StoreFromFloat(oRow, head * p.Dv + x, p.OutDtype, acc[t] * inv);
        }
    }
    if (lane == 0 && p.Lse.Valid()) {
        p.Lse.Row(head)[i] = m + log2f(l);
    }
}

// ---- backward: dQ ---------------------------------------------------------------------------
__global__ void __launch_bounds__(GEN_WARPS * 32) GenericBwdQKernel(TGenParams p)
{
    __shared__ float qs[GEN_WARPS][GEN_MAX_DIM];
    __shared__ float dos[GEN_WARPS][GEN_MAX_DIM];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int i = blockIdx.x * GEN_WARPS + warp;
    int head = blockIdx.y;
    if (i >= p.Len) {
        return;
    }
    float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
    float c = p.C * g;
    const uint8_t *qRow = p.Q.Row(i) + head * p.Dq;
    for (int x = lane; x < p.Dq; x += 32) {
        qs[warp][x] = Load8(qRow, x, p.QkDtype);
    }
    const void *doRow = p.DOut.Row(i);
    for (int x = lane; x < p.Dv; x += 32) {
        dos[warp][x] = LoadAsFloat(doRow, head * p.Dv + x, p.GradDtype);
    }
    __syncwarp();
    float sq = p.QScale.Valid() ? p.QScale.Row(head)[i] : p.QkVecScale;
    float rowMult = sq * c;
    float lse = p.Lse.Row(head)[i];
    float delta = p.DScale.Row(head)[i];
    float acc[GEN_ACC];
#pragma unroll
    for (int t = 0; t < GEN_ACC; ++t) {
        acc[t] = 0;
    }
    int blk = i / TSA_ATT_GROUP, r = i % TSA_ATT_GROUP;
    for (int gi = p.SpanPtr[blk]; gi < p.SpanPtr[blk + 1]; ++gi) {
        int s = max(p.Spans[gi].SpanStart[r], 0), f = min(p.Spans[gi].SpanFinish[r], p.KeyRows - 1);
        for (int j0 = s; j0 <= f; j0 += 32) {
            int j = j0 + lane;
            float t8 = 0;
            if (j <= f) {
                float sk = p.KScale.Row(head)[j];
                float dot = RowDot(qs[warp], p.K.Row(j) + head * p.Dq, p.Dq, p.QkDtype);
                float z = dot * sk * rowMult - p.Slope * (float)(i - j);
                float pij = exp2f(z - lse);
                float sv = p.VScale.Valid() ? p.VScale.Row(head)[j] : p.VVecScale;
                float dP = RowDot(dos[warp], p.V.Row(j) + head * p.Dv, p.Dv, p.VDtype) * sv;
                float dS = pij * (dP - delta) * c * kLog2;
                t8 = dS * sk;
            }
            int cnt = min(32, f - j0 + 1);
            for (int jj = 0; jj < cnt; ++jj) {
                float tj = __shfl_sync(0xffffffffu, t8, jj);
                const uint8_t *kRow = p.K.Row(j0 + jj) + head * p.Dq;
#pragma unroll
                for (int t = 0; t < GEN_ACC; ++t) {
                    int x = lane + 32 * t;
                    if (x < p.Dq) {
                        acc[t] += tj * Load8(kRow, x, p.QkDtype);
                    }
                }
            }
        }
    }
    void *dst = p.DQ.Row(i);
#pragma unroll
    for (int t = 0; t < GEN_ACC; ++t) {
        int x = lane + 32 * t;
        if (x < p.Dq) {
            StoreFromFloat(dst, head * p.Dq + x, p.GradDtype, acc[t] * p.GradMult);
        }
    }
}

// ---- backward: dK, dV over the transposed mask ----------------------------------------------
__global__ void __launch_bounds__(GEN_WARPS * 32) GenericBwdKVKernel(TGenParams p)
{
    __shared__ float ks[GEN_WARPS][GEN_MAX_DIM];
    __shared__ float vs[GEN_WARPS][GEN_MAX_DIM];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int j = blockIdx.x * GEN_WARPS + warp;
    int head = blockIdx.y;
    if (j >= p.Len) {
        return;
    }
    float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
    float c = p.C * g;
    const uint8_t *kRow = p.K.Row(j) + head * p.Dq;
    for (int x = lane; x < p.Dq; x += 32) {
        ks[warp][x] = Load8(kRow, x, p.QkDtype);
    }
    const uint8_t *vRow = p.V.Row(j) + head * p.Dv;
    for (int x = lane; x < p.Dv; x += 32) {
        vs[warp][x] = Load8(vRow, x, p.VDtype);
    }
    __syncwarp();
    float sk = p.KScale.Row(head)[j];
    float sv = p.VScale.Valid() ? p.VScale.Row(head)[j] : p.VVecScale;
    float accK[GEN_ACC], accV[GEN_ACC];
#pragma unroll
    for (int t = 0; t < GEN_ACC; ++t) {
        accK[t] = 0;
        accV[t] = 0;
    }
    int blk = j / TSA_ATT_GROUP, r = j % TSA_ATT_GROUP;
    for (int gi = p.RevSpanPtr[blk]; gi < p.RevSpanPtr[blk + 1]; ++gi) {
        int s = max(p.RevSpans[gi].SpanStart[r], 0), f = min(p.RevSpans[gi].SpanFinish[r], p.Len - 1);
        for (int i0 = s; i0 <= f; i0 += 32) {
            int i = i0 + lane;
            float tq = 0, pij = 0;
            if (i <= f) {
                float sq = p.QScale.Valid() ? p.QScale.Row(head)[i] : p.QkVecScale;
                float dot = RowDot(ks[warp], p.Q.Row(i) + head * p.Dq, p.Dq, p.QkDtype);
                float z = dot * sk * (sq * c) - p.Slope * (float)(i - j);
                pij = exp2f(z - p.Lse.Row(head)[i]);
                float dP = RowDotF(vs[warp], p.DOut.Row(i), head * p.Dv, p.Dv, p.GradDtype) * sv;
                float dS = pij * (dP - p.DScale.Row(head)[i]) * c * kLog2;
                tq = dS * sq;
            }
            int cnt = min(32, f - i0 + 1);
            for (int ii = 0; ii < cnt; ++ii) {
                float ti = __shfl_sync(0xffffffffu, tq, ii);
                float pi = __shfl_sync(0xffffffffu, pij, ii);
                const uint8_t *qRow = p.Q.Row(i0 + ii) + head * p.Dq;
                const void *doRow = p.DOut.Row(i0 + ii);
#pragma unroll
                for (int t = 0; t < GEN_ACC; ++t) {
                    int x = lane + 32 * t;
                    if (x < p.Dq) {
                        accK[t] += ti * Load8(qRow, x, p.QkDtype);
                    }
                    if (x < p.Dv) {
                        accV[t] += pi * LoadAsFloat(doRow, head * p.Dv + x, p.GradDtype);
                    }
                }
            }
        }
    }
    void *dk = p.DK.Row(j);
    void *dv = p.DV.Row(j);
#pragma unroll
    for (int t = 0; t < GEN_ACC; ++t) {
        int x = lane + 32 * t;
        if (x < p.Dq) {
            StoreFromFloat(dk, head * p.Dq + x, p.GradDtype, accK[t] * p.GradMult);
        }
        if (x < p.Dv) {
            StoreFromFloat(dv, head * p.Dv + x, p.GradDtype, accV[t] * p.GradMult);
        }
    }
}

int LaunchGenericFwd(const TGenParams &p, cudaStream_t stream)
{
    if (p.Len == 0) {
        return TSA_OK;
    }
    dim3 grid((p.Len + GEN_WARPS - 1) / GEN_WARPS, p.HeadCount);
    GenericFwdKernel<<<grid, GEN_WARPS * 32, 0, stream>>>(p);
    return CheckCuda(cudaGetLastError(), "generic forward launch");
}

int LaunchGenericBwd(const TGenParams &p, cudaStream_t stream)
{
    if (p.Len == 0) {
        return TSA_OK;
    }
    dim3 grid((p.Len + GEN_WARPS - 1) / GEN_WARPS, p.HeadCount);
    GenericBwdQKernel<<<grid, GEN_WARPS * 32, 0, stream>>>(p);
    GenericBwdKVKernel<<<grid, GEN_WARPS * 32, 0, stream>>>(p);
    return CheckCuda(cudaGetLastError(), "generic backward launch");
}

} // namespace tsa
