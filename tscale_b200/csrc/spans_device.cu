// Device-side generation of the grouped spans of window-causal masks (and of their transpose for the dK/dV pass):
// what tsa_group_window_spans computes on the host, written straight into device memory so that a training step
// neither waits for the host nor copies the mask.  Same records as GroupAttention<64,128> (code/gpt/att/att.h:95-181)
// applied to the spans of AddAttSpans (code/gpt/att/sliding_window.cpp:80-87) or to their TransposeAttention
// (code/gpt/att/att.cpp:26-56): window masks have the closed form
//   row i of a fragment [f0, f1]: attends [max(f0, i - window), i - 1];  is attended by [i + 1, min(f1, i + window)].
// One CTA; a warp builds the group of one 64-row block (two rows per lane); a block-wide scan of the "block has a group"
// flags gives groupPtr.  Integer work, a few microseconds for 2048 blocks.
#include "tsa_common.cuh"

namespace tsa {

constexpr int SPAN_THREADS = 1024;
constexpr int SPAN_WARPS = SPAN_THREADS / 32;
constexpr int kFarRightDev = 1000000000;

// fragStarts: fragCount + 1 ascending offsets, fragStarts[0] = 0, fragStarts[fragCount] = len
__device__ __forceinline__ void RowSpan(const int *fragStarts, int fragCount, int i, int window, int transposed, int *a, int *c)
{
    int lo = 0, hi = fragCount - 1; // last fragment whose start is <= i
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (fragStarts[mid] <= i) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    const int fragBase = fragStarts[lo], fragEnd = fragStarts[lo + 1] - 1;
    if (!transposed) {
        *a = (window > 0) ? max(fragBase, i - window) : fragBase;
        *c = i - 1;
    } else {
        *a = i + 1;
        *c = (window > 0) ? min(fragEnd, i + window) : fragEnd;
    }
}

__global__ void __launch_bounds__(SPAN_THREADS) GroupWindowSpansKernel(const int *fragStarts, int fragCount, int len, int window, int transposed,
    tsa_span_group *groups, int *groupPtr)
{
    __shared__ int warpTotals[SPAN_WARPS];
    __shared__ int carry;
    const int blocks = (len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        carry = 0;
        groupPtr[0] = 0;
    }
    __syncthreads();
    // passes of SPAN_THREADS blocks: thread tid owns the flag of block pass + tid, warp w builds blocks pass + 32 w .. + 31
    for (int pass = 0; pass < blocks; pass += SPAN_THREADS) {
        int myFlag = 0;
        // flags: every warp looks at its 32 blocks, one block per iteration, lane j keeps the flag of block j
        for (int j = 0; j < 32; ++j) {
            const int b = pass + warp * 32 + j;
            bool any = false;
            if (b < blocks) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int i = b * TSA_ATT_GROUP + half * 32 + lane;
                    if (i < len) {
                        int a, c;
                        RowSpan(fragStarts, fragCount, i, window, transposed, &a, &c);
                        any = any || a <= c;
                    }
                }
            }
            any = __any_sync(0xffffffffu, any);
            if (lane == j) {
                myFlag = any ? 1 : 0;
            }
        }
        // inclusive scan of the flags over the CTA
        int incl = myFlag;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) {
                incl += v;
            }
        }
        if (lane == 31) {
            warpTotals[warp] = incl;
        }
        __syncthreads();
        int warpBase = carry;
        for (int w = 0; w < warp; ++w) {
            warpBase += warpTotals[w];
        }
        const int b = pass + tid;
        if (b < blocks) {
            groupPtr[b + 1] = warpBase + incl;
        }
        // groups: rebuild block by block and write the record at its slot
        for (int j = 0; j < 32; ++j) {
            const int bb = pass + warp * 32 + j;
            const int flag = __shfl_sync(0xffffffffu, myFlag, j);
            const int slot = warpBase + __shfl_sync(0xffffffffu, incl, j) - 1;
            if (bb < blocks && flag) {
                int start = kFarRightDev, finish = 0;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int k = half * 32 + lane;
                    const int i = bb * TSA_ATT_GROUP + k;
                    int sa = kFarRightDev, sc = kFarRightDev - 1;
                    if (i < len) {
                        int a, c;
                        RowSpan(fragStarts, fragCount, i, window, transposed, &a, &c);
                        if (a <= c) {
                            sa = a;
                            sc = c;
                            start = min(start, a);
                            finish = max(finish, c);
                        }
                    }
                    groups[slot].SpanStart[k] = sa;
                    groups[slot].SpanFinish[k] = sc;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    start = min(start, __shfl_xor_sync(0xffffffffu, start, o));
                    finish = max(finish, __shfl_xor_sync(0xffffffffu, finish, o));
                }
                if (lane == 0) {
                    groups[slot].Start = start / TSA_ATT_ALIGN * TSA_ATT_ALIGN;
                    groups[slot].Finish = finish / TSA_ATT_ALIGN * TSA_ATT_ALIGN;
                }
            }
        }
        __syncthreads();
        if (tid == SPAN_THREADS - 1) {
            carry = warpBase + incl;
        }
        __syncthreads();
    }
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) int tsa_group_window_spans_device(const int *fragStarts, int fragCount, int len, int window,
    int transposed, int maxGroups, tsa_span_group *groups, int *groupPtr, tsa_stream_t stream)
{
    TSA_REQUIRE(fragCount >= 0 && len >= 0, "tsa_group_window_spans_device: negative size");
    TSA_REQUIRE(groupPtr != nullptr, "tsa_group_window_spans_device: null groupPtr");
    const int blocks = (len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP;
    if (fragCount == 0 || len == 0) {
        return CheckCuda(cudaMemsetAsync(groupPtr, 0, sizeof(int) * (blocks + 1), (cudaStream_t)stream), "clearing groupPtr");
    }
    TSA_REQUIRE(fragStarts && groups, "tsa_group_window_spans_device: null buffer");
    TSA_REQUIRE(maxGroups >= blocks, "tsa_group_window_spans_device: room for %d groups needed (one per 64-row block), %d given", blocks, maxGroups);
    GroupWindowSpansKernel<<<1, SPAN_THREADS, 0, (cudaStream_t)stream>>>(fragStarts, fragCount, len, window, transposed, groups, groupPtr);
    return CheckCuda(cudaGetLastError(), "tsa_group_window_spans_device launch");
}
