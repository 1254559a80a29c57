// Device-side building blocks shared by the engine: activation layout, epilogue description,
// and the launchers of every kernel.  All launchers enqueue on the given stream and return
// the CUDA error of the launch.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace kb {

enum DType { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
inline size_t dtypeSize(int dt) { return dt == DT_F32 ? 4 : 2; }

// Activation layout ("padded rows").  A batch of boards is one matrix of rows x channels; the row of
// point (n,y,x) is n*PB + y*RW + x with RW = X+1 and PB = (Y+1)*RW.  Column X of every line and line Y of
// every board are padding that always holds zeros in tensors that feed a convolution, so the 8 neighbours
// of a point are at fixed row offsets (dy*RW + dx) and a 3x3 convolution is nine row-shifted GEMMs.
// rowsPad = rows rounded up to a multiple of 256 (two MMA tiles of 128 rows: a CTA pair works on both).
struct Geom {
  int X, Y, RW, PB, S;
  int n;        // boards in this batch
  int rows;     // n * PB
  int rowsPad;  // rows rounded up to 256
};

inline Geom makeGeom(int X, int Y, int n) {
  Geom g;
  g.X = X; g.Y = Y; g.RW = X + 1; g.PB = (Y + 1) * (X + 1); g.S = X * Y; g.n = n;
  g.rows = n * g.PB;
  g.rowsPad = (g.rows + 255) / 256 * 256;
  return g;
}

// What a convolution does with each accumulator v[row][c] (c in [0,outC)):
//   v += biasNC[n][c]            (per-board bias: global-feature bias, gpool bias)   if biasNC
//   v += residual[row][c]   (resMask: v = v*mask[row] + residual[row][c], the transformer blocks' masked residual add,
//                            eigenbackend.cpp:1573-1582)                              if residual
//   outRaw[row][c - rawC0] = v                     for c in [rawC0, rawC1)           if outRaw
//   outAct[row][c - actC0] = mask[row]==1 ? act(v*scale[c-actC0] + bias[c-actC0]) : 0
//                                                  for c in [actC0, actC1)           if outAct
// The second form is the NEXT layer's batch norm + activation + board mask (eigenbackend.cpp:739-763)
// applied while the accumulator is still on chip.
// Epilogue::act value used only by the tensor-core convolution for the merged FFN up|gate projection whose output
// channels are interleaved in groups of 16 (16 "up" channels, then their 16 "gate" channels): instead of the two
// halves it writes h = silu(up) * gate (eigenbackend.cpp:1660-1672), 16 values per 32 accumulator columns, to outAct
// ([rows][actStride], channel (c - actC0) / 2).  scale/bias/mask are not used.
constexpr int KB_ACT_SWIGLU_PAIRS = 100;
// Epilogue::act value used only by the tensor-core convolution for the merged Q|K|V projection of an attention block:
// the rotary embedding (eigenbackend.cpp:1415-1451) is applied to the query and key heads while the accumulators are
// still fp32 registers, so the attention kernel finds Q and K rotated and rounded once.  There is no activated output;
// outRaw receives the rotated values.  See ropeFreq / ropeC1 of Epilogue.
constexpr int KB_ACT_ROPE_QK = 101;

struct Epilogue {
  const float* biasNC = nullptr;
  const void* residual = nullptr;
  int resStride = 0;
  int resMask = 0;
  void* outRaw = nullptr;
  int rawStride = 0, rawC0 = 0, rawC1 = 0;
  void* outAct = nullptr;
  int actStride = 0, actC0 = 0, actC1 = 0;
  const float* scale = nullptr;
  const float* bias = nullptr;
  int act = 0;
  const float* mask = nullptr;
  // Row-wise RMS normalisation folded around a convolution (pre-norm transformer blocks, eigenbackend.cpp:867-918;
  // tensor-core convolution with the shared-memory staged epilogue only).  A producer of the residual stream stores
  // partial sums of squares of every row of its raw output: sumsqOut[slot * sumsqRowStride + row], one slot per
  // (channel tile, epilogue warp of the row quarter), each written by exactly one thread, so the result does not depend
  // on any ordering.  A consumer adds rowSumsqSlots partials in slot order and multiplies each accumulator row by
  // rsqrt(sum/C + eps) (0 where the mask is 0) before anything else; with the norm's gain folded into its weights that
  // equals conv(rmsnorm(x)).  convTcRowSumSlots gives the producer's slot count.
  float* sumsqOut = nullptr;
  const float* rowSumsq = nullptr;
  int rowSumsqSlots = 0;
  int sumsqRowStride = 0;
  float rowInvC = 0.0f, rowEps = 0.0f;
  // act == KB_ACT_ROPE_QK: output channels [0, ropeC1) are the query and key heads (ropeC1 <= 1024, a multiple of 32).
  // Channel pair (2i, 2i+1), at board point (x,y), turns by the angle x * ropeFreq[2i] + y * ropeFreq[2i+1]
  // (desc.cpp:1212-1275: the head's frequencies, expanded per output channel pair by the caller).  Sine and cosine come
  // from the special-function unit (absolute error about 2e-6 at the largest angles of a 19x19 board with frequencies
  // up to 1, two orders of magnitude below the rounding of the stored fp16/bf16 value).
  const float* ropeFreq = nullptr;
  int ropeC1 = 0;
};

// --- SIMT kernels (any dtype) ---------------------------------------------------------------------

// Packs NNEvaluator-style inputs into the padded-rows layout, applying the per-row board symmetry
// (nninputs.cpp:529-597) and producing mask (= input channel 0, eigenbackend.cpp:2169) and maskSum.
// spatial: [n][Y][X][inC] fp32.  dst: [rowsPad][dstStride] (channels >= inC are left zero).
cudaError_t launchPackInput(
  cudaStream_t st, int dt, const float* spatial, const int32_t* symmetry, int inC, void* dst, int dstStride,
  float* mask, float* maskSum, Geom g);

// Generic convolution on CUDA cores: any odd kernel size, any channel counts, fp32 accumulate.
// in: [rowsPad][inStride]; w: [kY*kX][inC][outC] in the activation dtype.
cudaError_t launchConvSimt(
  cudaStream_t st, int dt, const void* in, int inStride, int inC, const void* w, int outC, int kY, int kX,
  Geom g, const Epilogue& ep);

// out[r][oc] (+)= act(sum_ic in[r][ic]*w[ic][oc] + bias[oc]); fp32, small row counts (heads, gpool bias, metadata encoder).
cudaError_t launchMatMulSmall(
  cudaStream_t st, const float* in, int inC, const float* w, int outC, const float* bias, int act, float* out, int rows,
  int accumulate = 0);

// Masked global pooling (eigenbackend.cpp:152-197).  in: [rowsPad][inStride] (channels c0..c0+C), already
// activated and masked.  out: [n][3*C] fp32.  valueHead selects the third statistic.
cudaError_t launchGPool(
  cudaStream_t st, int dt, const void* in, int inStride, int c0, int C, const float* mask, const float* maskSum,
  float* out, int valueHead, Geom g);

// out[row][c] = mask ? act((in[row][c] + biasNC[n][c]) * scale[c] + bias[c]) : 0   (addNCBiasInplace + BN)
cudaError_t launchBiasBnAct(
  cudaStream_t st, int dt, const void* in, int inStride, const float* biasNC, const float* scale, const float* bias,
  int act, const float* mask, void* out, int outStride, int C, Geom g);

// The three steps between the first and the last convolution of a global-pooling block in one launch: pooled statistics
// of gIn (activated gpool branch, Cg channels), board bias = stats [3*Cg] x w (stored output-major, [Cr][3*Cg]), out = mask ? act((rIn + bias) *
// scale + bias) : 0 over the regular branch (Cr channels).  Reduced precision with 8-channel-aligned tensors only.
bool gpoolMidEligible(int dt, int Cg, int gStride, int Cr, int rStride, int outStride);
cudaError_t launchGPoolMid(
  cudaStream_t st, int dt, const void* gIn, int gStride, int Cg, const void* rIn, int rStride, int Cr, const float* w,
  const float* scale, const float* bias, int act, const float* mask, const float* maskSum, void* out, int outStride, Geom g);

// Stand-alone batch norm + activation + mask (first layer of a block whose input was not produced by one
// of our convolutions, and the single-layer test entry points).
cudaError_t launchBnAct(
  cudaStream_t st, int dtIn, const void* in, int inStride, const float* scale, const float* bias, int act,
  const float* mask, int dtOut, void* out, int outStride, int C, Geom g);

// Final 1x1 convolutions of the heads: policy = p2Conv(pAct), ownership = ownConv(vAct), written to the
// caller-facing fp32 arrays with the inverse board symmetry.  pAct: [rowsPad][pStride] (P1 channels),
// vAct: [rowsPad][vStride] channels v0..v0+V1.  w2: [P1][policyC] fp32, wOwn: [V1] fp32.
cudaError_t launchHeadFinal(
  cudaStream_t st, int dt, const void* pAct, int pStride, int P1, const float* w2, int policyC, const void* vAct,
  int vStride, int v0, int V1, const float* wOwn, const int32_t* symmetry, float* policy, float* ownership, Geom g);

// Everything of the heads after their first convolutions in one launch, one CTA per board (reduced precision, channel
// counts that are multiples of 8).  pRaw [rowsPad][P1]: policy p1 convolution output; gv [rowsPad][G1+V1]: activated g1 |
// v1 outputs.  Matmul weights are fp32, stored output-major ([out][in]); passH = 0: no pass MLP (wPass is then [Pc][3*G1]).  Outputs: policy
// [n][S][Pc] and ownership [n][S] in the caller's frame (symmetry may be NULL), pass [n][Pc], value [n][Vc], score [n][Sv].
struct HeadsTailArgs {
  const void* pRaw; const void* gv;
  int P1, G1, V1, Pc, Vc, Sv, V2, passH;
  const float* wGB;
  const float* wPass; const float* bPass; int passAct; const float* wPass2;
  const float* pScale; const float* pBias; int pAct;
  const float* w2; const float* wOwn;
  const float* wV2; const float* bV2; int v2Act;
  const float* wV3; const float* bV3; const float* wSV; const float* bSV;
  const float* mask; const float* maskSum; const int32_t* symmetry;
  float* outPolicy; float* outOwnership; float* outPass; float* outValue; float* outScore;
};
bool headsTailEligible(int dt, const HeadsTailArgs& a);
cudaError_t launchHeadsTail(cudaStream_t st, int dt, const HeadsTailArgs& a, Geom g);

// Layout conversion for the single-layer entry points: [n][Y][X][C] fp32 <-> padded rows of dtype dt.
cudaError_t launchToPadded(cudaStream_t st, int dt, const float* src, int C, void* dst, int dstStride, Geom g);
cudaError_t launchFromPadded(cudaStream_t st, int dt, const void* src, int srcStride, int C, float* dst, Geom g);
// mask [n][Y][X] fp32 -> padded mask + maskSum
cudaError_t launchMaskToPadded(cudaStream_t st, const float* src, float* mask, float* maskSum, Geom g);

// --- Tensor-core convolution (fp16 / bf16, sm_100a tcgen05) ------------------------------------------

struct ConvTcPlan;  // opaque: tensor maps + tile configuration for one convolution
// True if the tensor-core kernel can run this convolution shape.
bool convTcEligible(int dt, int inC, int outC, int kY, int kX);
// True if a 1x1 convolution inC -> outC takes the staged epilogue that supports sumsqOut / rowSumsq.
bool convTcRowNormEligible(int dt, int inC, int outC);
// Number of partial-sum slots a convolution of this shape writes per row when Epilogue::sumsqOut is set.
int convTcRowSumSlots(int k, int inC, int outC);
// the slot count of a planned convolution whose epilogue has been set (it depends on the epilogue-warp variant chosen)
int convTcPlanRowSumSlots(const struct ConvTcPlan* p);
// True if the tensor-core kernel can run the merged up|gate projection (inC -> 2*F, interleaved) with the SwiGLU epilogue.
bool convTcSwigluEligible(int dt, int inC, int F);
// the merged Q|K|V projection can apply the rotary embedding in its epilogue (Epilogue::act == KB_ACT_ROPE_QK)
bool convTcRopeEligible(int dt, int inC, int outC, int ropeC1);
// in: [rowsPadMax][inStride] activations, w: [kY*kX][outC][inC] in dtype dt (K-major per tap).
ConvTcPlan* convTcCreate(
  int dt, const void* in, int inStride, int inC, const void* w, int outC, int kY, int kX, int X, int Y, int rowsPadMax);
void convTcDestroy(ConvTcPlan* p);
// Binds the epilogue (output/residual tensors) to the plan; must be called once before the first launch.
bool convTcSetEpilogue(ConvTcPlan* p, const Epilogue& ep);
// Per-tile dependencies between two tensor-core convolutions launched one after the other (see ConvTcArgs::depCtr):
// `done` = this launch's counters (one per 128-row tile, zero before the launch), `wait` / `waitPlan` = counters and
// plan of the convolution launched immediately before it.
struct ConvTcDeps {
  uint32_t* done = nullptr;
  const uint32_t* wait = nullptr;
  const ConvTcPlan* waitPlan = nullptr;
};
bool convTcDepsCapable(const ConvTcPlan* p);
int convTcKernelSize(const ConvTcPlan* p);
// True if the tile table marks this shape for multi-layer launches.
bool convTcChainPreferred(const ConvTcPlan* p);
int convTcDoneCount(const ConvTcPlan* p);
int convTcGridSize(const ConvTcPlan* p, const Geom& g);
cudaError_t launchConvTc(cudaStream_t st, const ConvTcPlan* p, Geom g, const Epilogue& ep, int* statusWord, const ConvTcDeps* deps = nullptr);

// The closing 1x1 convolution of a nested bottleneck block fused with the opening 1x1 convolution of the next one
// (kb_conv_fused.cu): stream += w1 * in1; raw2 = w2 * act(stream * scale1 + bias1) * mask; act2 = act(raw2 * scale2 +
// bias2) * mask.  The activated stream itself is not written anywhere.  Dense tensors, fp16 / bf16.
struct ConvPostPrePlan;
bool convPostPreEligible(int dt, int Cm, int Ct, int Cn);
ConvPostPrePlan* convPostPreCreate(
  int dt, const void* in1, int Cm, const void* w1, void* stream, int Ct, const float* scale1, const float* bias1, int act1,
  const void* w2, void* raw2, void* act2, int Cn, const float* scale2, const float* bias2, int act2code, const float* mask,
  int rowsPadMax);
void convPostPreDestroy(ConvPostPrePlan* p);
cudaError_t launchConvPostPre(cudaStream_t st, const ConvPostPrePlan* p, Geom g, int* statusWord);

// Self-test of the bounded device-side waits: a kernel waits (limitNs, at most one second) on a barrier nothing arrives
// at, gives up, and records code 199 in the status word.
cudaError_t launchWaitTimeoutSelfTest(cudaStream_t st, int* statusWord, unsigned long long limitNs);

// Several consecutive tensor-core convolutions as ONE persistent launch whose tiles hand over through per-tile counters
// (kb_conv_tc.cu, "chain").  members[i].done: counter array of layer i (one per 128-row tile of rowsPadMax, zeroed by the
// caller before every launch), needed for every layer but the last.  Every plan must have had its epilogue bound.
struct ConvChainPlan;
struct ConvChainMember {
  const ConvTcPlan* plan = nullptr;
  Epilogue ep;
  uint32_t* done = nullptr;
};
int convTcTileWidth(const ConvTcPlan* p);
bool convChainEligible(const ConvTcPlan* p, const Epilogue& ep);
ConvChainPlan* convChainCreate(const ConvChainMember* members, int n);
void convChainDestroy(ConvChainPlan* c);
cudaError_t launchConvChain(cudaStream_t st, const ConvChainPlan* c, Geom g, int* statusWord);

}  // namespace kb

namespace kb {

// --- Transformer pieces (CUDA cores; the projections themselves run through the convolution path as 1x1) ---------

// Per-position RMS norm over channels (eigenbackend.cpp:867-1022): out = x * rsqrt(mean_c(x^2) + eps) * gamma[c] (+ beta[c]),
// optional SiLU, masked rows -> 0.  beta may be NULL.  in/out: [rowsPad][stride] of dtype dt.
cudaError_t launchRmsNorm(
  cudaStream_t st, int dt, const void* in, int inStride, const float* gamma, const float* beta, float eps, int silu,
  const float* mask, void* out, int outStride, int C, Geom g);

// Spatial RMS norm (eigenbackend.cpp:979-1020): one scale per board over all on-board points and channels.
// scratch: [n] floats.
cudaError_t launchSpatialRmsNorm(
  cudaStream_t st, int dt, const void* in, int inStride, const float* gamma, const float* beta, float eps, int silu,
  const float* mask, void* out, int outStride, int C, float* scratch, Geom g);

// Rotary embedding on interleaved channel pairs (eigenbackend.cpp:1415-1451), in place on `heads` heads of `dim`
// channels starting at column c0 of buf.  cosT/sinT: [tableHeads][dim/2][S]; head h uses table h*tableHeads/heads.
cudaError_t launchRope(
  cudaStream_t st, int dt, void* buf, int stride, int c0, int heads, int dim, const float* cosT, const float* sinT,
  int tableHeads, Geom g);

// Masked softmax attention over the board points of each board (eigenbackend.cpp:1455-1560).  qkv: [rowsPad][stride]
// with Q at column qOff (heads*dq), K at kOff (kvHeads*dq), V at vOff (kvHeads*dv).  out: [rowsPad][outStride]
// (heads*dv); rows of masked or padding points are written as zeros.
// relBias (or NULL): learned relative-position bias [heads][2*relY-1][2*relX-1], added to the scaled score of query
// (yq,xq) and key (yk,xk) at [head][yk-yq+relY-1][xk-xq+relX-1].
// The kernel keeps K, V and a row block of the scores of one board in shared memory: true if a board of X x Y fits.
bool attentionFits(int X, int Y, int dq, int dv);
cudaError_t launchAttention(
  cudaStream_t st, int dt, const void* qkv, int stride, int qOff, int kOff, int vOff, int heads, int kvHeads, int dq, int dv,
  const float* mask, void* out, int outStride, Geom g, const float* relBias = nullptr, int relY = 0, int relX = 0);

// SwiGLU (eigenbackend.cpp:1660-1672): out[r][c] = silu(in[r][c]) * in[r][C + c].
cudaError_t launchSwiGLU(cudaStream_t st, int dt, const void* in, int inStride, void* out, int outStride, int C, Geom g);

// Tensor-core attention (fp16/bf16, head dimension 64, boards whose Y*(X+1) rows fit 384 keys).
struct AttnTcPlan;
bool attentionTcEligible(int dt, int dq, int dv, int X, int Y, int stride, int qOff, int kOff, int vOff, int outStride);
AttnTcPlan* attentionTcCreate(int dt, const void* qkv, int stride, int totalCols, int rowsPadMax);
void attentionTcDestroy(AttnTcPlan* p);
// ropeX/ropeY (or NULL): the rotary embedding is applied to Q and K inside the kernel, so the QKV matrix holds the
// unrotated projections.  The angle of pair p at point (x,y) is ax(p,x) + ay(p,y); ropeX [tableHeads][32][X] and ropeY
// [tableHeads][32][Y] hold (cos, sin) of the two parts.
cudaError_t launchAttentionTc(
  cudaStream_t st, const AttnTcPlan* p, int qOff, int kOff, int vOff, int heads, int kvHeads, const float* mask, void* out,
  int outStride, Geom g, int* statusWord, const float2* ropeX, const float2* ropeY, int tableHeads,
  const float* relBias = nullptr, int relY = 0, int relX = 0, int pipelined = 1);
// pipelined: without in-kernel rotation the work runs on persistent CTAs with a dedicated issuing warp (0: one CTA per
// (board, head), as with rotation; same bits).
// relBias (or NULL): learned relative-position bias as for launchAttention; the kernel keeps one head's table in shared
// memory, which bounds it to KB_ATTN_TC_REL_MAX entries.
constexpr int KB_ATTN_TC_REL_MAX = 1536;

}  // namespace kb
