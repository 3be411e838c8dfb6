// Device-side TransposeAttention and GroupAttention for arbitrary span lists: what tsa_transpose_attention and
// tsa_group_attention compute on the host (code/gpt/att/att.cpp:26-56, code/gpt/att/att.h:95-181), for masks that are
// already in device memory (document-boundary masks, masks built by a kernel), so that a step neither waits for the host
// nor copies the mask.  Integer work; every result is bit-identical to the host helpers'.
//
// Transpose without walking (row, key) pairs.  Key `to` is attended by the maximal runs of consecutive rows that have
// it in a span.  A run starts at row i exactly on the keys that row i attends and row i - 1 does not, and ends at row i
// on the keys that row i attends and row i + 1 does not, so per row only the interval differences
//   spans(i) \ spans(i - 1)   and   spans(i) \ spans(i + 1)
// are needed (two sorted lists walked once).  The number of runs over a key is the number of start intervals covering
// it (difference array + scan); every start interval then drops its row into the lists of the keys it covers, every end
// interval likewise, and because both kinds are visited in ascending row order per key after a small sort, the k-th
// start pairs with the k-th end.  Rows' spans must be sorted by start and disjoint, as AddAttSpans produces them.
#include "att_internal.cuh"

namespace tsa {

namespace {

constexpr int SCAN_THREADS = 1024;

struct TIv {
    int A, B;
};

// spans of one row clipped to [0, len - 1]; empty ones are skipped by Next()
struct TRowSpans {
    const int *Spans;
    int Pos, End, Len;
    __device__ TRowSpans(const int *spans, const int *spanPtr, int row, int len) : Spans(spans), Pos(0), End(0), Len(len)
    {
        if (row >= 0 && row < len) {
            Pos = spanPtr[row];
            End = spanPtr[row + 1];
        }
    }
    __device__ bool Next(TIv *iv)
    {
        while (Pos < End) {
            const int a = max(0, Spans[2 * Pos]), b = min(Len - 1, Spans[2 * Pos + 1]);
            ++Pos;
            if (a <= b) {
                iv->A = a;
                iv->B = b;
                return true;
            }
        }
        return false;
    }
};

// calls emit(a, b) for every maximal interval of spans(row) that spans(other) does not cover
template <class TEmit>
__device__ void RowDifference(const int *spans, const int *spanPtr, int row, int other, int len, TEmit emit)
{
    TRowSpans mine(spans, spanPtr, row, len), theirs(spans, spanPtr, other, len);
    TIv cover;
    bool haveCover = theirs.Next(&cover);
    TIv iv;
    while (mine.Next(&iv)) {
        int cur = iv.A;
        for (;;) {
            while (haveCover && cover.B < cur) {
                haveCover = theirs.Next(&cover);
            }
            if (!haveCover || cover.A > iv.B) {
                emit(cur, iv.B);
                break;
            }
            if (cover.A > cur) {
                emit(cur, cover.A - 1);
            }
            cur = cover.B + 1;
            if (cur > iv.B) {
                break;
            }
        }
    }
}

// pass 0: counts of start / end intervals per row;  pass 1: the intervals themselves at the scanned offsets
template <int PASS>
__global__ void __launch_bounds__(256) RunEdgeKernel(int len, const int *spans, const int *spanPtr, int *cntS, int *cntE, const int *offS,
    const int *offE, int *ivS, int *ivE, int *diff)
{
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= len) {
        return;
    }
    int nS = 0, nE = 0;
    const int baseS = PASS ? offS[row] : 0, baseE = PASS ? offE[row] : 0;
    RowDifference(spans, spanPtr, row, row - 1, len, [&](int a, int b) {
        if (PASS) {
            ivS[3 * (baseS + nS)] = a;
            ivS[3 * (baseS + nS) + 1] = b;
            ivS[3 * (baseS + nS) + 2] = row;
            atomicAdd(diff + a, 1);
            atomicAdd(diff + b + 1, -1);
        }
        ++nS;
    });
    RowDifference(spans, spanPtr, row, row + 1, len, [&](int a, int b) {
        if (PASS) {
            ivE[3 * (baseE + nE)] = a;
            ivE[3 * (baseE + nE) + 1] = b;
            ivE[3 * (baseE + nE) + 2] = row;
        }
        ++nE;
    });
    if (!PASS) {
        cntS[row] = nS;
        cntE[row] = nE;
    }
}

// exclusive scan of src[0..n) into dst[0..n], dst[n] = total; one CTA.  inclusiveFirst: src holds differences and the
// value of element i is the inclusive prefix sum (runs over key i), which is then scanned exclusively.
__global__ void __launch_bounds__(SCAN_THREADS) ScanKernel(const int *src, int n, int *dst, int fromDifferences, int *total)
{
    __shared__ long long part[SCAN_THREADS];
    __shared__ int carryIn[SCAN_THREADS];
    const int tid = threadIdx.x;
    const int per = (n + SCAN_THREADS - 1) / SCAN_THREADS;
    const int i0 = min(n, tid * per), i1 = min(n, i0 + per);
    if (fromDifferences) {
        // first the values: inclusive prefix sums of the differences
        int s = 0;
        for (int i = i0; i < i1; ++i) {
            s += src[i];
        }
        carryIn[tid] = s;
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int k = 0; k < SCAN_THREADS; ++k) {
                const int v = carryIn[k];
                carryIn[k] = run;
                run += v;
            }
        }
        __syncthreads();
    }
    long long sum = 0;
    {
        int level = fromDifferences ? carryIn[tid] : 0;
        for (int i = i0; i < i1; ++i) {
            level = fromDifferences ? level + src[i] : src[i];
            sum += level;
        }
    }
    part[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        long long run = 0;
        for (int k = 0; k < SCAN_THREADS; ++k) {
            const long long v = part[k];
            part[k] = run;
            run += v;
        }
        dst[n] = (int)min(run, (long long)0x7fffffff);
        if (total) {
            *total = dst[n];
        }
    }
    __syncthreads();
    long long run = part[tid];
    int level = fromDifferences ? carryIn[tid] : 0;
    for (int i = i0; i < i1; ++i) {
        level = fromDifferences ? level + src[i] : src[i];
        dst[i] = (int)min(run, (long long)0x7fffffff);
        run += level;
    }
}

// every start (end) interval drops its row into the start (end) slots of the keys it covers; one warp per interval
__global__ void __launch_bounds__(256) FillRunsKernel(const int *iv, const int *ivCount, const int *resSpanPtr, int *fill, int *resSpans, int which,
    int maxSpans, const int *total, int *count)
{
    if (*total > maxSpans) {
        if (blockIdx.x == 0 && threadIdx.x == 0 && which == 0) {
            count[1] = 1; // the caller's arrays are too small: nothing is written
        }
        return;
    }
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int n = *ivCount;
    for (int k = warp; k < n; k += warps) {
        const int a = iv[3 * k], b = iv[3 * k + 1], row = iv[3 * k + 2];
        for (int to = a + lane; to <= b; to += 32) {
            const int slot = atomicAdd(fill + to, 1);
            resSpans[2 * (resSpanPtr[to] + slot) + which] = row;
        }
    }
}

// per key: its start rows and its end rows in ascending order (insertion sort; the lists are short)
__global__ void __launch_bounds__(256) SortRunsKernel(int len, const int *resSpanPtr, int *resSpans, int maxSpans, const int *total)
{
    if (*total > maxSpans) {
        return;
    }
    const int to = blockIdx.x * blockDim.x + threadIdx.x;
    if (to >= len) {
        return;
    }
    const int p0 = resSpanPtr[to], n = resSpanPtr[to + 1] - p0;
    for (int which = 0; which < 2; ++which) {
        int *base = resSpans + 2 * p0 + which;
        for (int i = 1; i < n; ++i) {
            const int v = base[2 * i];
            int j = i - 1;
            while (j >= 0 && base[2 * j] > v) {
                base[2 * (j + 1)] = base[2 * j];
                --j;
            }
            base[2 * (j + 1)] = v;
        }
    }
}

// ---- grouping: one CTA of 64 threads per 64-row block, thread k = row k of the block
__global__ void __launch_bounds__(TSA_ATT_GROUP) GroupRoundsKernel(int len, const int *spanPtr, int *rounds)
{
    __shared__ int mx;
    const int row = blockIdx.x * TSA_ATT_GROUP + threadIdx.x;
    if (threadIdx.x == 0) {
        mx = 0;
    }
    __syncthreads();
    if (row < len) {
        atomicMax(&mx, spanPtr[row + 1] - spanPtr[row]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        rounds[blockIdx.x] = mx;
    }
}

__global__ void __launch_bounds__(TSA_ATT_GROUP) GroupFillKernel(int len, const int *spans, const int *spanPtr, const int *groupPtr, int maxGroups,
    tsa_span_group *groups, int *count)
{
    const int kFarRight = 1000000000;
    __shared__ int lo, hi;
    const int blocks = (len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP;
    if (groupPtr[blocks] > maxGroups) {
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            count[1] = 1;
        }
        return;
    }
    const int k = threadIdx.x, row = blockIdx.x * TSA_ATT_GROUP + k;
    const int p0 = row < len ? spanPtr[row] : 0, n = row < len ? spanPtr[row + 1] - p0 : 0;
    const int g0 = groupPtr[blockIdx.x], rounds = groupPtr[blockIdx.x + 1] - g0;
    for (int r = 0; r < rounds; ++r) {
        if (k == 0) {
            lo = kFarRight;
            hi = 0;
        }
        __syncthreads();
        // round r holds the r-th span (by start; equal starts keep their order) of every row that still has one: the
        // rank of a span among its row's spans is found by counting, which is a stable sort for the short lists of a row
        int s = kFarRight, f = kFarRight - 1;
        if (r < n) {
            for (int c = 0; c < n; ++c) {
                const int cs = spans[2 * (p0 + c)];
                int rank = 0;
                for (int o = 0; o < n; ++o) {
                    const int os = spans[2 * (p0 + o)];
                    rank += (os < cs || (os == cs && o < c)) ? 1 : 0;
                }
                if (rank == r) {
                    s = cs;
                    f = spans[2 * (p0 + c) + 1];
                    break;
                }
            }
            atomicMin(&lo, s);
            atomicMax(&hi, f);
        }
        tsa_span_group *g = groups + g0 + r;
        g->SpanStart[k] = s;
        g->SpanFinish[k] = f;
        __syncthreads();
        if (k == 0) {
            g->Start = lo / TSA_ATT_ALIGN * TSA_ATT_ALIGN;
            g->Finish = hi / TSA_ATT_ALIGN * TSA_ATT_ALIGN;
        }
        __syncthreads();
    }
}

size_t RoundUpInts(size_t n)
{
    return (n + 63) & ~(size_t)63;
}

} // namespace

} // namespace tsa

using namespace tsa;

// workspace (ints): cntS, cntE [len], offS, offE [len + 1], diff [len + 2], fillS, fillE [len], totals [8], start and end
// intervals 3 x 2 x maxInputSpans each (a row adds at most spans(i) + spans(i +- 1) intervals)
extern "C" __attribute__((visibility("default"))) size_t tsa_transpose_attention_device_workspace_bytes(int len, int maxInputSpans)
{
    if (len < 0 || maxInputSpans < 0) {
        return 0;
    }
    const size_t L = RoundUpInts((size_t)len + 2);
    return (7 * L + 64 + 2 * RoundUpInts(6 * (size_t)maxInputSpans + 6)) * sizeof(int);
}

extern "C" __attribute__((visibility("default"))) int tsa_transpose_attention_device(int len, const int *spans, const int *spanPtr, int maxInputSpans,
    int maxSpans, int *resSpans, int *resSpanPtr, int *count, void *workspace, size_t workspaceBytes, tsa_stream_t stream)
{
    TSA_REQUIRE(len >= 0 && spanPtr && resSpanPtr && count && (resSpans || maxSpans == 0), "tsa_transpose_attention_device: null argument");
    TSA_REQUIRE(spans || maxInputSpans == 0, "tsa_transpose_attention_device: null spans");
    const size_t need = tsa_transpose_attention_device_workspace_bytes(len, maxInputSpans);
    TSA_REQUIRE(workspace && workspaceBytes >= need && (uintptr_t)workspace % 16 == 0, "tsa_transpose_attention_device: workspace of %zu bytes needed, %zu given",
        need, workspaceBytes);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t L = RoundUpInts((size_t)len + 2), I = RoundUpInts(6 * (size_t)maxInputSpans + 6);
    int *w = (int *)workspace;
    int *cntS = w, *cntE = w + L, *offS = w + 2 * L, *offE = w + 3 * L, *diff = w + 4 * L, *fillS = w + 5 * L, *fillE = w + 6 * L;
    int *totals = w + 7 * L;
    int *ivS = totals + 64, *ivE = ivS + I;
    int rc = CheckCuda(cudaMemsetAsync(diff, 0, 3 * L * sizeof(int), s), "clearing the transpose workspace");
    if (rc == TSA_OK) {
        rc = CheckCuda(cudaMemsetAsync(count, 0, 2 * sizeof(int), s), "clearing the transpose counters");
    }
    if (rc != TSA_OK) {
        return rc;
    }
    const int rowBlocks = (len + 255) / 256;
    if (len > 0) {
        RunEdgeKernel<0><<<rowBlocks, 256, 0, s>>>(len, spans, spanPtr, cntS, cntE, nullptr, nullptr, nullptr, nullptr, nullptr);
    }
    ScanKernel<<<1, SCAN_THREADS, 0, s>>>(cntS, len, offS, 0, totals + 0);
    ScanKernel<<<1, SCAN_THREADS, 0, s>>>(cntE, len, offE, 0, totals + 1);
    if (len > 0) {
        RunEdgeKernel<1><<<rowBlocks, 256, 0, s>>>(len, spans, spanPtr, cntS, cntE, offS, offE, ivS, ivE, diff);
    }
    // runs over key `to` = inclusive prefix sum of diff; resSpanPtr = exclusive scan of the runs; count[0] = total
    ScanKernel<<<1, SCAN_THREADS, 0, s>>>(diff, len, resSpanPtr, 1, count);
    if (len > 0) {
        FillRunsKernel<<<148 * 4, 256, 0, s>>>(ivS, totals + 0, resSpanPtr, fillS, resSpans, 0, maxSpans, count, count);
        FillRunsKernel<<<148 * 4, 256, 0, s>>>(ivE, totals + 1, resSpanPtr, fillE, resSpans, 1, maxSpans, count, count);
        SortRunsKernel<<<rowBlocks, 256, 0, s>>>(len, resSpanPtr, resSpans, maxSpans, count);
    }
    return CheckCuda(cudaGetLastError(), "tsa_transpose_attention_device launches");
}

extern "C" __attribute__((visibility("default"))) size_t tsa_group_attention_device_workspace_bytes(int len)
{
    return len < 0 ? 0 : RoundUpInts((size_t)(len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP + 2) * sizeof(int);
}

extern "C" __attribute__((visibility("default"))) int tsa_group_attention_device(int len, const int *spans, const int *spanPtr, int maxGroups,
    tsa_span_group *groups, int *groupPtr, int *count, void *workspace, size_t workspaceBytes, tsa_stream_t stream)
{
    TSA_REQUIRE(len >= 0 && spanPtr && groupPtr && count && (groups || maxGroups == 0), "tsa_group_attention_device: null argument");
    const size_t need = tsa_group_attention_device_workspace_bytes(len);
    TSA_REQUIRE(workspace && workspaceBytes >= need && (uintptr_t)workspace % 16 == 0, "tsa_group_attention_device: workspace of %zu bytes needed, %zu given",
        need, workspaceBytes);
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP;
    int *rounds = (int *)workspace;
    int rc = CheckCuda(cudaMemsetAsync(count, 0, 2 * sizeof(int), s), "clearing the group counters");
    if (rc != TSA_OK) {
        return rc;
    }
    if (blocks > 0) {
        GroupRoundsKernel<<<blocks, TSA_ATT_GROUP, 0, s>>>(len, spanPtr, rounds);
    }
    ScanKernel<<<1, SCAN_THREADS, 0, s>>>(rounds, blocks, groupPtr, 0, count);
    if (blocks > 0) {
        GroupFillKernel<<<blocks, TSA_ATT_GROUP, 0, s>>>(len, spans, spanPtr, groupPtr, maxGroups, groups, count);
    }
    return CheckCuda(cudaGetLastError(), "tsa_group_attention_device launches");
}
