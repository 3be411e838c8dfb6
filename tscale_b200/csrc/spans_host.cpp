// Host-side preparation of the attention mask in the form the kernels take: per-row inclusive key
// spans (CSR), their transpose for the dK/dV pass, and the grouped form of 64-row blocks.
// Behaviour follows the reference's AddAttSpans (code/gpt/att/sliding_window.cpp:80-87),
// TransposeAttention (code/gpt/att/att.cpp:26-56) and GroupAttention<64,128> (code/gpt/att/att.h:95-181);
// the algorithms are our own: the transpose is an event sweep over an interval set instead of a walk
// over every (row, key) pair, and window masks have a closed form that never enumerates spans.
#include "tsa.h"
#include <algorithm>
#include <map>
#include <utility>
#include <vector>

namespace {

const int kFarRight = 1000000000;

struct TBlockGroups {
    // rows x rounds spans of one 64-row block
    std::vector<std::pair<int, int>> Rows[TSA_ATT_GROUP];
};

void InitGroup(tsa_span_group *g)
{
    g->Start = kFarRight;
    g->Finish = 0;
    for (int k = 0; k < TSA_ATT_GROUP; ++k) {
        g->SpanStart[k] = kFarRight;
        g->SpanFinish[k] = kFarRight - 1;
    }
}

void CloseGroup(tsa_span_group *g)
{
    g->Start = g->Start / TSA_ATT_ALIGN * TSA_ATT_ALIGN;
    g->Finish = g->Finish / TSA_ATT_ALIGN * TSA_ATT_ALIGN;
}

// set of disjoint runs [a, b] of active row indices
class TRunSet {
    std::map<int, int> Runs; // start -> finish
public:
    void Insert(int x)
    {
        auto next = Runs.lower_bound(x);
        bool joinNext = next != Runs.end() && next->first == x + 1;
        bool joinPrev = false;
        auto prev = next;
        if (next != Runs.begin()) {
            prev = std::prev(next);
            if (prev->second >= x) {
                return; // already present
            }
            joinPrev = prev->second == x - 1;
        }
        if (joinPrev && joinNext) {
            prev->second = next->second;
            Runs.erase(next);
        } else if (joinPrev) {
            prev->second = x;
        } else if (joinNext) {
            int fin = next->second;
            Runs.erase(next);
            Runs[x] = fin;
        } else {
            Runs[x] = x;
        }
    }
    void Erase(int x)
    {
        auto it = Runs.upper_bound(x);
        if (it == Runs.begin()) {
            return;
        }
        --it;
        int a = it->first, b = it->second;
        if (x > b) {
            return;
        }
        Runs.erase(it);
        if (a <= x - 1) {
            Runs[a] = x - 1;
        }
        if (x + 1 <= b) {
            Runs[x + 1] = b;
        }
    }
    const std::map<int, int> &Get() const { return Runs; }
};

} // namespace

extern "C" __attribute__((visibility("default"))) int tsa_make_window_spans(int fragCount, const int *fragLens, int window, int maxSpans, int *spans, int *spanPtr)
{
    if (fragCount < 0 || (fragCount > 0 && !fragLens) || !spanPtr) {
        return 0;
    }
    long long total = 0;
    for (int pass = 0; pass < 2; ++pass) {
        int base = 0, ptr = 0, row = 0;
        spanPtr[0] = 0;
        for (int f = 0; f < fragCount; ++f) {
            for (int i = base; i < base + fragLens[f]; ++i) {
                int lo = (window > 0) ? std::max(base, i - window) : base;
                if (i - 1 >= lo) {
                    if (pass == 1) {
                        spans[2 * ptr] = lo;
                        spans[2 * ptr + 1] = i - 1;
                    }
                    ++ptr;
                }
                spanPtr[++row] = ptr;
            }
            base += fragLens[f];
        }
        total = ptr;
        if (pass == 0 && (total > maxSpans || !spans)) {
            return total > maxSpans ? -(int)total : (int)total;
        }
    }
    return (int)total;
}

extern "C" __attribute__((visibility("default"))) int tsa_transpose_attention(int len, const int *spans, const int *spanPtr, int maxSpans, int *resSpans, int *resSpanPtr)
{
    if (len < 0 || !spanPtr || !resSpanPtr) {
        return 0;
    }
    // events: row `from` becomes active at key Start and inactive after key Finish
    std::vector<std::vector<int>> addAt(len + 1), dropAt(len + 1);
    for (int from = 0; from < len; ++from) {
        for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
            int a = std::max(0, spans[2 * s]), b = std::min(len - 1, spans[2 * s + 1]);
            if (a <= b) {
                addAt[a].push_back(from);
                dropAt[b + 1].push_back(from);
            }
        }
    }
    TRunSet active;
    long long total = 0;
    resSpanPtr[0] = 0;
    for (int to = 0; to < len; ++to) {
        for (int from : dropAt[to]) {
            active.Erase(from);
        }
        for (int from : addAt[to]) {
            active.Insert(from);
        }
        for (const auto &run : active.Get()) {
            if (total < maxSpans && resSpans) {
                resSpans[2 * total] = run.first;
                resSpans[2 * total + 1] = run.second;
            }
            ++total;
        }
        resSpanPtr[to + 1] = (int)total;
    }
    return total > maxSpans ? -(int)total : (int)total;
}

extern "C" __attribute__((visibility("default"))) int tsa_group_attention(int len, const int *spans, const int *spanPtr, int maxGroups, tsa_span_group *groups, int *groupPtr)
{
    if (len < 0 || !spanPtr || !groupPtr) {
        return 0;
    }
    int blocks = (len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP;
    long long total = 0;
    groupPtr[0] = 0;
    std::vector<std::pair<int, int>> rowSpans[TSA_ATT_GROUP];
    for (int b = 0; b < blocks; ++b) {
        size_t rounds = 0;
        for (int k = 0; k < TSA_ATT_GROUP; ++k) {
            rowSpans[k].clear();
            int from = b * TSA_ATT_GROUP + k;
            if (from < len) {
                for (int s = spanPtr[from]; s < spanPtr[from + 1]; ++s) {
                    rowSpans[k].push_back(std::make_pair(spans[2 * s], spans[2 * s + 1]));
                }
                std::stable_sort(rowSpans[k].begin(), rowSpans[k].end(),
                    [](const std::pair<int, int> &x, const std::pair<int, int> &y) { return x.first < y.first; });
                rounds = std::max(rounds, rowSpans[k].size());
            }
        }
        // round r holds the r-th span of every row that still has one
        for (size_t r = 0; r < rounds; ++r) {
            if (total < maxGroups && groups) {
                tsa_span_group *g = groups + total;
                InitGroup(g);
                for (int k = 0; k < TSA_ATT_GROUP; ++k) {
                    if (r < rowSpans[k].size()) {
                        g->SpanStart[k] = rowSpans[k][r].first;
                        g->SpanFinish[k] = rowSpans[k][r].second;
                        g->Start = std::min(g->Start, rowSpans[k][r].first);
                        g->Finish = std::max(g->Finish, rowSpans[k][r].second);
                    }
                }
                CloseGroup(g);
            }
            ++total;
        }
        groupPtr[b + 1] = (int)total;
    }
    return total > maxGroups ? -(int)total : (int)total;
}

extern "C" __attribute__((visibility("default"))) int tsa_group_window_spans(int fragCount, const int *fragLens, int window, int transposed, int maxGroups,
    tsa_span_group *groups, int *groupPtr)
{
    if (fragCount < 0 || (fragCount > 0 && !fragLens) || !groupPtr) {
        return 0;
    }
    long long len = 0;
    for (int f = 0; f < fragCount; ++f) {
        len += fragLens[f];
    }
    int blocks = (int)((len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP);
    long long total = 0;
    groupPtr[0] = 0;
    int frag = 0, fragBase = 0;
    for (int b = 0; b < blocks; ++b) {
        tsa_span_group g;
        InitGroup(&g);
        bool any = false;
        for (int k = 0; k < TSA_ATT_GROUP; ++k) {
            int i = b * TSA_ATT_GROUP + k;
            if (i >= len) {
                break;
            }
            while (i >= fragBase + fragLens[frag]) {
                fragBase += fragLens[frag];
                ++frag;
            }
            int fragEnd = fragBase + fragLens[frag] - 1;
            int a, c;
            if (!transposed) {
                a = (window > 0) ? std::max(fragBase, i - window) : fragBase;
                c = i - 1;
            } else {
                a = i + 1;
                c = (window > 0) ? std::min(fragEnd, i + window) : fragEnd;
            }
            if (a <= c) {
                g.SpanStart[k] = a;
                g.SpanFinish[k] = c;
                g.Start = std::min(g.Start, a);
                g.Finish = std::max(g.Finish, c);
                any = true;
            }
        }
        if (any) {
            if (total < maxGroups && groups) {
                CloseGroup(&g);
                groups[total] = g;
            }
            ++total;
        }
        groupPtr[b + 1] = (int)total;
    }
    return total > maxGroups ? -(int)total : (int)total;
}

// ---- partition of one batch over the GPUs of a box --------------------------------------------------
// The reference splits a batch over its devices by fragments and gives every device its own context, host thread and
// stream (TMultiComputeContext, code/gpt/compute/gpt_cuda.cu:1478-1738; batch split code/gpt/train_ctx/backprop.cpp:10-23).
// Here the unit is one (fragment, head) pair, numbered fragment-major: unit = fragment * heads + head.  Units are
// independent (spans never cross fragments, heads never mix), so a contiguous block of units per rank needs no exchange
// on the way in.
extern "C" __attribute__((visibility("default"))) int tsa_shard_range(int units, int world, int rank, int *begin, int *end)
{
    if (units < 0 || world <= 0 || rank < 0 || rank >= world || !begin || !end) {
        return TSA_BAD_ARG;
    }
    const int base = units / world, rem = units % world;
    *begin = rank * base + std::min(rank, rem);
    *end = *begin + base + (rank < rem ? 1 : 0);
    return TSA_OK;
}

// A contiguous unit range as at most three rectangles (fragment range x head range), in unit order: the tail of the
// first fragment, the whole fragments in the middle, the head of the last fragment.  Each rectangle is one tsa_att_fwd
// call on the rectangle's rows and head columns.  Returns the number of rectangles written, or a negative tsa_status.
extern "C" __attribute__((visibility("default"))) int tsa_shard_rects(int begin, int end, int heads, tsa_shard_rect *rects)
{
    if (begin < 0 || end < begin || heads <= 0 || !rects) {
        return -TSA_BAD_ARG;
    }
    int n = 0;
    int cur = begin;
    while (cur < end && n < 3) {
        const int frag = cur / heads, head = cur % heads;
        tsa_shard_rect r;
        r.frag_begin = frag;
        r.head_begin = head;
        if (head != 0 || end - cur < heads) {
            // part of one fragment
            r.frag_end = frag + 1;
            r.head_end = std::min(heads, head + (end - cur));
        } else {
            r.frag_end = frag + (end - cur) / heads;
            r.head_end = heads;
        }
        cur += (r.frag_end - r.frag_begin) * (r.head_end - r.head_begin);
        rects[n++] = r;
    }
    return n;
}
