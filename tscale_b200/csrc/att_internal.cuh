// Parameter blocks and launch functions shared by the attention translation units.
#pragma once
#include "tsa_common.cuh"

namespace tsa {

constexpr int GEN_WARPS = 4;
constexpr int GEN_MAX_DIM = 256;
constexpr int GEN_ACC = GEN_MAX_DIM / 32;

struct TGenParams {
    int Len;          // rows with spans (lenAttTiles * 64 clipped to buffers)
    int KeyRows;      // rows of qv / v: spans are clipped to [0, KeyRows)
    int HeadCount;
    int Dq, Dv;
    int QkDtype, VDtype, OutDtype, GradDtype;
    float C;          // attDotScale (without *g)
    const float *GlobalScale;
    float QkVecScale, VVecScale;
    float Slope;
    float GradMult;
    P2D<uint8_t> Q, K, V;
    P2D<float> QScale, KScale, VScale;
    P2D<char> Out;
    P2D<char> OutCopy[TSA_MAX_OUT_COPIES]; // further destinations of the forward's output (same shape as Out; peer-GPU memory allowed)
    int OutCopies = 0;
    // consumer fused into the forward (tsa_att_fwd_kv): combiner key rows bf16 [len][H*D], combiner input bf16 [len][H*4D]
    P2D<char> KvK, KvOut;
    float KvMult = 1.0f;
    P2D<float> Lse;
    P2D<char> DOut;
    P2D<float> DScale;
    P2D<char> DQ, DK, DV;
    const tsa_span_group *Spans;
    const int *SpanPtr;
    const tsa_span_group *RevSpans;
    const int *RevSpanPtr;
};


int LaunchGenericFwd(const TGenParams &p, cudaStream_t stream);
int LaunchGenericBwd(const TGenParams &p, cudaStream_t stream);
int LaunchDScale(int outDtype, int gradDtype, tsa_ptr2d out, tsa_ptr2d dOut, tsa_ptr2d dScale,
    int headCount, int headDimV, int len, cudaStream_t stream);

// parity hook of the int8 forward: where the kernel stores the raw s32 scores of one key tile as it read them
struct TFwdDump {
    int32_t *Dst = nullptr; // [128][128] int32 in device memory, null = off
    int Head = 0, QTile = 0, Tile = 0;
    long long WaitCycles = 0; // self-test: bound of the forward's barrier waits (0: the production bound)
    int WithholdTile = -1;    // self-test: a key tile copy every CTA requests but never issues (-1: none)
};
int LaunchBoundedWaitSelfTest(long long limitCycles, int *statusWord, cudaStream_t stream);
void SetFwdScoreDump(const TFwdDump &d);

// tcgen05 forward (att_fwd_sm100.cu).  Returns TSA_UNSUPPORTED when the configuration is outside
// the tensor-core path (the caller then uses the generic kernels).
bool Sm100FwdSupports(const tsa_att_cfg *cfg, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v);
size_t Sm100FwdWorkspaceBytes(const tsa_att_cfg *cfg, int headCount, int keyRows);
int LaunchSm100Fwd(const tsa_att_cfg *cfg, const TGenParams &p, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v,
    int lenAttTiles, int keyRows, void *workspace, int *statusWord, cudaStream_t stream);

// tcgen05 backward (att_bwd_sm100.cu): two launches of one kernel (dQ pass, dK/dV pass) after widening the stored
// vectors to bf16 in the workspace
bool Sm100BwdSupports(const tsa_att_cfg *cfg, int headCount);
size_t Sm100BwdWorkspaceBytes(int headCount, int headDim, int rows);
int LaunchSm100Bwd(const tsa_att_cfg *cfg, const TGenParams &p, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v, tsa_ptr2d dOut,
    int lenAttTiles, void *workspace, int *statusWord, cudaStream_t stream);

} // namespace tsa
