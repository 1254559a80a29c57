/* CPU oracle: fp32 restatement of the reference's Eigen backend.  TEST INFRASTRUCTURE ONLY
 * (see kata_oracle.h).  Each function cites the reference code it follows
 * (paths relative to the reference's cpp/ directory).
 *
 * Layout: every activation tensor is NHWC, stored as rows of C floats, row index
 * r = n*S + y*X + x with S = X*Y.  Convolutions are computed directly (the reference
 * uses Winograd for 3x3/5x5, neuralnet/eigenbackend.cpp:335-412, which is the same
 * function up to fp32 rounding).
 */
#include "kata_oracle.h"
#include "../include/kb_modelblob.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

using std::vector;
using kbblob::Reader;
using kbblob::Record;

namespace {

thread_local std::string g_lastError;

// ------------------------------------------------------------------------------------------------
// Storage emulation (ko_set_storage_emulation): NOT part of the reference's arithmetic.  It rounds selected tensors to
// fp16 or bf16 where a reduced-precision backend stores them, everything else staying fp32, so that tests can measure
// how far ANY backend with that storage scheme must move from the fp32 result (the floor that the tolerance tests add
// their bound to).  Off by default; set once before a forward pass, not while one runs.
int g_emuType = 0;   // 0 off, 1 fp16, 2 bf16
int g_emuFlags = 0;  // KO_EMU_CONV_INPUTS | KO_EMU_STREAMS
// Where the rounding sits (it mirrors a backend whose convolution epilogues write both the updated stream and the next
// layer's activated tensor from the fp32 accumulator): activated tensors are rounded where a convolution (or a pooling
// layer) reads them; a residual stream is rounded just before the next branch is added to it, so the norm that follows
// an update still sees the value before rounding; intermediate sums that such a backend stores before a per-board bias
// is known (the regular path of a gpool block, the policy head's p1) are rounded at that point.

inline float roundBf16(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if((u & 0x7f800000u) == 0x7f800000u) return x;
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  std::memcpy(&x, &u, 4);
  return x;
}
inline float roundStorage(float x) {
  if(g_emuType == 1) return (float)(_Float16)x;
  if(g_emuType == 2) return roundBf16(x);
  return x;
}
void roundTensor(float* p, size_t count) {
#pragma omp parallel for schedule(static)
  for(size_t i = 0; i < count; i++) p[i] = roundStorage(p[i]);
}
inline bool emuOn(int flag) { return g_emuType != 0 && (g_emuFlags & flag) != 0; }

struct Fail : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// ------------------------------------------------------------------------------------------------
// Activations.  neuralnet/eigenbackend.cpp:749-760 (BatchNormLayer::apply) and :783-810 (ActivationLayer).

inline float applyAct(float x, int act) {
  switch(act) {
    case KB_ACT_IDENTITY: return x;
    case KB_ACT_RELU: return x > 0.0f ? x : 0.0f;
    case KB_ACT_MISH: {
      // x * tanh(log1p(exp(min(x,20))) + (max(x,20) - 20))
      float sp = log1pf(expf(std::min(x, 20.0f))) + (std::max(x, 20.0f) - 20.0f);
      return x * tanhf(sp);
    }
    case KB_ACT_SILU: return x / (expf(-x) + 1.0f);
    case KB_ACT_MISH_SCALE8: {
      // x * tanh(softplus(8x)); neuralnet/desc.cpp:402-432.  The Eigen backend never sees this
      // activation; it is provided so that scale-8 transformed descs can be evaluated too.
      float x8 = 8.0f * x;
      float sp = log1pf(expf(std::min(x8, 20.0f))) + (std::max(x8, 20.0f) - 20.0f);
      return x * tanhf(sp);
    }
    default: throw Fail("unknown activation code " + std::to_string(act));
  }
}

// ------------------------------------------------------------------------------------------------
// Layers

struct Conv {
  int kY = 0, kX = 0, inC = 0, outC = 0;
  vector<float> w;  // repacked to [y][x][ic][oc]

  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_CONV, 6, "CONV");
    kY = r.ints[0]; kX = r.ints[1]; inC = r.ints[2]; outC = r.ints[3];
    int dilY = r.ints[4], dilX = r.ints[5];
    if(kY <= 0 || kX <= 0 || (kY % 2) != 1 || (kX % 2) != 1) throw Fail("conv: kernel sizes must be odd and positive");
    if(inC <= 0 || outC <= 0) throw Fail("conv: channels must be positive");
    // The Eigen backend rejects dilation != 1 (neuralnet/eigenbackend.cpp:325-330).
    if(dilY != 1 || dilX != 1) throw Fail("conv: dilation other than 1 is not supported");
    if((size_t)r.nFloats != (size_t)kY * kX * inC * outC) throw Fail("conv: wrong number of weights");
    w.resize(r.nFloats);
    // blob order is the reference desc order [oc][ic][y][x] (neuralnet/desc.h:23)
    for(int oc = 0; oc < outC; oc++)
      for(int ic = 0; ic < inC; ic++)
        for(int y = 0; y < kY; y++)
          for(int x = 0; x < kX; x++)
            w[(((size_t)y * kX + x) * inC + ic) * outC + oc] = r.floats[(((size_t)oc * inC + ic) * kY + y) * kX + x];
  }

  // out (+)= cross-correlation of in with w, zero padded, stride 1.
  // neuralnet/eigenbackend.cpp:565-703 (ConvLayer::apply; `accumulate` adds into the output).
  void apply(const float* in, float* out, int n, int X, int Y, bool accumulate) const {
    const int S = X * Y;
    const int padY = kY / 2, padX = kX / 2;
    const int PB = 4;
    vector<float> roundedIn;
    // the stored residual stream is what the next update adds to; the value before rounding fed the norm that follows it
    if(accumulate && emuOn(KO_EMU_STREAMS)) roundTensor(out, (size_t)n * S * outC);
    if(emuOn(KO_EMU_CONV_INPUTS)) {
      roundedIn.assign(in, in + (size_t)n * S * inC);
      roundTensor(roundedIn.data(), roundedIn.size());
      in = roundedIn.data();
    }
#pragma omp parallel for collapse(2) schedule(static)
    for(int b = 0; b < n; b++) {
      for(int y = 0; y < Y; y++) {
        vector<float> accBuf((size_t)PB * outC);
        for(int x0 = 0; x0 < X; x0 += PB) {
          const int np = std::min(PB, X - x0);
          std::fill(accBuf.begin(), accBuf.end(), 0.0f);
          for(int dy = 0; dy < kY; dy++) {
            int iy = y + dy - padY;
            if(iy < 0 || iy >= Y) continue;
            for(int dx = 0; dx < kX; dx++) {
              const float* wt = &w[((size_t)dy * kX + dx) * inC * outC];
              const float* src[PB];
              for(int p = 0; p < PB; p++) {
                int ix = x0 + p + dx - padX;
                src[p] = (p < np && ix >= 0 && ix < X) ? in + ((size_t)b * S + (size_t)iy * X + ix) * inC : nullptr;
              }
              for(int ic = 0; ic < inC; ic++) {
                const float* wrow = wt + (size_t)ic * outC;
                for(int p = 0; p < PB; p++) {
                  if(src[p] == nullptr) continue;
                  const float v = src[p][ic];
                  float* acc = &accBuf[(size_t)p * outC];
#pragma omp simd
                  for(int oc = 0; oc < outC; oc++) acc[oc] += v * wrow[oc];
                }
              }
            }
          }
          for(int p = 0; p < np; p++) {
            float* dst = out + ((size_t)b * S + (size_t)y * X + x0 + p) * outC;
            const float* acc = &accBuf[(size_t)p * outC];
            if(accumulate) for(int oc = 0; oc < outC; oc++) dst[oc] += acc[oc];
            else for(int oc = 0; oc < outC; oc++) dst[oc] = acc[oc];
          }
        }
      }
    }
  }
};

struct BN {
  int C = 0, act = 0;
  vector<float> scale, bias;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_BN, 2, "BN");
    C = r.ints[0]; act = r.ints[1];
    if(C <= 0 || r.nFloats != (uint32_t)(2 * C)) throw Fail("bn: wrong number of floats");
    scale.assign(r.floats, r.floats + C);
    bias.assign(r.floats + C, r.floats + 2 * C);
  }
  // neuralnet/eigenbackend.cpp:739-763: out = mask==1 ? act(in*scale+bias) : 0
  void apply(const float* in, float* out, const float* mask, size_t rows) const {
#pragma omp parallel for schedule(static)
    for(size_t r = 0; r < rows; r++) {
      const float* src = in + r * C;
      float* dst = out + r * C;
      if(mask[r] == 1.0f) for(int c = 0; c < C; c++) dst[c] = applyAct(src[c] * scale[c] + bias[c], act);
      else for(int c = 0; c < C; c++) dst[c] = 0.0f;
    }
  }
};

struct MatMul {
  int inC = 0, outC = 0;
  vector<float> w;  // [ic][oc]
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_MATMUL, 2, "MATMUL");
    inC = r.ints[0]; outC = r.ints[1];
    if(inC <= 0 || outC <= 0 || (size_t)r.nFloats != (size_t)inC * outC) throw Fail("matmul: wrong number of weights");
    w.assign(r.floats, r.floats + r.nFloats);
  }
  // neuralnet/eigenbackend.cpp:814-841: out[row][oc] = sum_ic in[row][ic] * w[ic][oc]
  void apply(const float* in, float* out, size_t rows) const {
#pragma omp parallel for schedule(static) if(rows > 64)
    for(size_t r = 0; r < rows; r++) {
      const float* src = in + r * inC;
      float* dst = out + r * outC;
      for(int oc = 0; oc < outC; oc++) dst[oc] = 0.0f;
      for(int ic = 0; ic < inC; ic++) {
        const float v = src[ic];
        const float* wrow = &w[(size_t)ic * outC];
#pragma omp simd
        for(int oc = 0; oc < outC; oc++) dst[oc] += v * wrow[oc];
      }
    }
  }
};

struct MatBias {
  int C = 0;
  vector<float> b;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_MATBIAS, 1, "MATBIAS");
    C = r.ints[0];
    if(C <= 0 || r.nFloats != (uint32_t)C) throw Fail("matbias: wrong number of floats");
    b.assign(r.floats, r.floats + C);
  }
  // neuralnet/eigenbackend.cpp:843-862
  void apply(float* mat, size_t rows) const {
    for(size_t r = 0; r < rows; r++)
      for(int c = 0; c < C; c++) mat[r * C + c] += b[c];
  }
};

int loadAct(Reader& rd) {
  Record r = rd.expect(KB_TAG_ACT, 1, "ACT");
  return r.ints[0];
}

// neuralnet/eigenbackend.cpp:137-148 addNCBiasInplace: x[n][s][c] += bias[n][c]
void addNCBias(float* x, const float* bias, int n, int S, int C) {
#pragma omp parallel for schedule(static)
  for(int b = 0; b < n; b++)
    for(int s = 0; s < S; s++) {
      float* row = x + ((size_t)b * S + s) * C;
      const float* br = bias + (size_t)b * C;
      for(int c = 0; c < C; c++) row[c] += br[c];
    }
}

// neuralnet/eigenbackend.cpp:152-177 poolRowsGPool
void poolRowsGPool(const float* in, float* out, const float* mask, const float* maskSum, int n, int S, int C) {
#pragma omp parallel for schedule(static)
  for(int b = 0; b < n; b++) {
    for(int c = 0; c < C; c++) {
      float s = 0.0f;
      float m = -1.0f;
      for(int p = 0; p < S; p++) {
        float x = in[((size_t)b * S + p) * C + c];
        s += x;
        float maskVal = mask[(size_t)b * S + p];
        m = std::max(m, x + (maskVal - 1.0f));
      }
      float div = maskSum[b];
      float sqrtdiv = sqrtf(div);
      float mean = s / div;
      out[(size_t)b * 3 * C + c] = mean;
      out[(size_t)b * 3 * C + C + c] = mean * (sqrtdiv - 14.0f) * 0.1f;
      out[(size_t)b * 3 * C + 2 * C + c] = m;
    }
  }
}

// neuralnet/eigenbackend.cpp:179-197 poolRowsValueHead
void poolRowsValueHead(const float* in, float* out, const float* maskSum, int n, int S, int C) {
#pragma omp parallel for schedule(static)
  for(int b = 0; b < n; b++) {
    for(int c = 0; c < C; c++) {
      float s = 0.0f;
      for(int p = 0; p < S; p++) s += in[((size_t)b * S + p) * C + c];
      float div = maskSum[b];
      float sqrtdiv = sqrtf(div);
      float mean = s / div;
      out[(size_t)b * 3 * C + c] = mean;
      out[(size_t)b * 3 * C + C + c] = mean * (sqrtdiv - 14.0f) * 0.1f;
      out[(size_t)b * 3 * C + 2 * C + c] = mean * ((sqrtdiv - 14.0f) * (sqrtdiv - 14.0f) * 0.01f - 0.1f);
    }
  }
}

// neuralnet/eigenbackend.cpp:867-918 TransformerRMSNormLayer
struct TRMSNorm {
  int C = 0;
  float eps = 0.0f;
  vector<float> weight;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_TRMSNORM, 1, "TRMSNORM");
    C = r.ints[0];
    if(C <= 0 || r.nFloats != (uint32_t)(C + 1)) throw Fail("trmsnorm: wrong number of floats");
    eps = r.floats[0];
    weight.assign(r.floats + 1, r.floats + 1 + C);
  }
  void apply(const float* in, float* out, const float* mask, size_t rows) const {
#pragma omp parallel for schedule(static)
    for(size_t r = 0; r < rows; r++) {
      const float* src = in + r * C;
      float* dst = out + r * C;
      if(mask[r] == 0.0f) { for(int c = 0; c < C; c++) dst[c] = 0.0f; continue; }
      float sumSq = 0.0f;
      for(int c = 0; c < C; c++) sumSq += src[c] * src[c];
      float rms = 1.0f / sqrtf(sumSq / (float)C + eps);
      for(int c = 0; c < C; c++) dst[c] = src[c] * rms * weight[c];
    }
  }
};

// neuralnet/eigenbackend.cpp:923-1022 RMSNormLayer (trunk tip)
struct RMSNorm {
  int C = 0, spatial = 0, act = 0;
  float eps = 0.0f;
  vector<float> gamma, beta;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_RMSNORM, 3, "RMSNORM");
    C = r.ints[0]; spatial = r.ints[1]; act = r.ints[2];
    if(C <= 0 || r.nFloats != (uint32_t)(2 * C + 1)) throw Fail("rmsnorm: wrong number of floats");
    eps = r.floats[0];
    gamma.assign(r.floats + 1, r.floats + 1 + C);
    beta.assign(r.floats + 1 + C, r.floats + 1 + 2 * C);
  }
  void apply(const float* in, float* out, const float* mask, int n, int S) const {
#pragma omp parallel for schedule(static)
    for(int b = 0; b < n; b++) {
      float sampleRms = 0.0f;
      if(spatial) {
        float sumSq = 0.0f;
        int count = 0;
        for(int p = 0; p < S; p++) {
          if(mask[(size_t)b * S + p] == 0.0f) continue;
          const float* src = in + ((size_t)b * S + p) * C;
          for(int c = 0; c < C; c++) sumSq += src[c] * src[c];
          count++;
        }
        float totalElts = (float)count * (float)C;
        sampleRms = 1.0f / sqrtf(sumSq / totalElts + eps);
      }
      for(int p = 0; p < S; p++) {
        const float* src = in + ((size_t)b * S + p) * C;
        float* dst = out + ((size_t)b * S + p) * C;
        if(mask[(size_t)b * S + p] == 0.0f) { for(int c = 0; c < C; c++) dst[c] = 0.0f; continue; }
        float rms = sampleRms;
        if(!spatial) {
          float sumSq = 0.0f;
          for(int c = 0; c < C; c++) sumSq += src[c] * src[c];
          rms = 1.0f / sqrtf(sumSq / (float)C + eps);
        }
        for(int c = 0; c < C; c++) {
          float v = src[c] * rms * gamma[c] + beta[c];
          // Only SiLU is applied here by the reference (eigenbackend.cpp:974-975, 1012-1013).
          if(act == KB_ACT_SILU) v = v / (1.0f + expf(-v));
          dst[c] = v;
        }
      }
    }
  }
};

// ------------------------------------------------------------------------------------------------
// Blocks

struct Ctx {
  int n, X, Y, S;
  const float* mask;     // [n*S]
  const float* maskSum;  // [n]
  size_t rows() const { return (size_t)n * S; }
};

struct Block {
  virtual ~Block() {}
  // trunk is updated in place; [n*S][C]
  virtual void apply(const Ctx& cx, float* trunk) const = 0;
  virtual int channels() const = 0;
};

std::unique_ptr<Block> loadBlock(Reader& rd);

// neuralnet/eigenbackend.cpp:1091-1134 ResidualBlock
struct OrdinaryBlock final : Block {
  BN preBN; Conv conv1; BN midBN; Conv conv2;
  void load(Reader& rd) {
    rd.expect(KB_TAG_BLOCK_ORDINARY, 0, "BLOCK_ORDINARY");
    preBN.load(rd); conv1.load(rd); midBN.load(rd); conv2.load(rd);
    if(preBN.C != conv1.inC || conv1.outC != midBN.C || midBN.C != conv2.inC || conv2.outC != preBN.C)
      throw Fail("ordinary block: channel mismatch");
  }
  int channels() const override { return preBN.C; }
  void apply(const Ctx& cx, float* trunk) const override {
    vector<float> scratch(cx.rows() * preBN.C), mid(cx.rows() * conv1.outC), midScratch(cx.rows() * conv1.outC);
    preBN.apply(trunk, scratch.data(), cx.mask, cx.rows());
    conv1.apply(scratch.data(), mid.data(), cx.n, cx.X, cx.Y, false);
    midBN.apply(mid.data(), midScratch.data(), cx.mask, cx.rows());
    conv2.apply(midScratch.data(), trunk, cx.n, cx.X, cx.Y, true);
  }
};

// neuralnet/eigenbackend.cpp:1138-1218 GlobalPoolingResidualBlock
struct GPoolBlock final : Block {
  BN preBN; Conv regularConv; Conv gpoolConv; BN gpoolBN; MatMul gpoolToBias; BN midBN; Conv finalConv;
  void load(Reader& rd) {
    rd.expect(KB_TAG_BLOCK_GPOOL, 0, "BLOCK_GPOOL");
    preBN.load(rd); regularConv.load(rd); gpoolConv.load(rd); gpoolBN.load(rd);
    gpoolToBias.load(rd); midBN.load(rd); finalConv.load(rd);
    if(preBN.C != regularConv.inC || preBN.C != gpoolConv.inC || gpoolConv.outC != gpoolBN.C ||
       gpoolToBias.inC != 3 * gpoolBN.C || gpoolToBias.outC != regularConv.outC ||
       midBN.C != regularConv.outC || finalConv.inC != midBN.C || finalConv.outC != preBN.C)
      throw Fail("gpool block: channel mismatch");
  }
  int channels() const override { return preBN.C; }
  void apply(const Ctx& cx, float* trunk) const override {
    const size_t rows = cx.rows();
    vector<float> scratch(rows * preBN.C), regularOut(rows * regularConv.outC), regularScratch(rows * regularConv.outC);
    vector<float> gpoolOut(rows * gpoolConv.outC), gpoolOut2(rows * gpoolConv.outC);
    vector<float> gpoolConcat((size_t)cx.n * 3 * gpoolConv.outC), gpoolBias((size_t)cx.n * regularConv.outC);
    preBN.apply(trunk, scratch.data(), cx.mask, rows);
    regularConv.apply(scratch.data(), regularOut.data(), cx.n, cx.X, cx.Y, false);
    if(emuOn(KO_EMU_CONV_INPUTS)) roundTensor(regularOut.data(), regularOut.size());  // stored before the pooled bias is known
    gpoolConv.apply(scratch.data(), gpoolOut.data(), cx.n, cx.X, cx.Y, false);
    gpoolBN.apply(gpoolOut.data(), gpoolOut2.data(), cx.mask, rows);
    if(emuOn(KO_EMU_CONV_INPUTS)) roundTensor(gpoolOut2.data(), gpoolOut2.size());
    poolRowsGPool(gpoolOut2.data(), gpoolConcat.data(), cx.mask, cx.maskSum, cx.n, cx.S, gpoolConv.outC);
    gpoolToBias.apply(gpoolConcat.data(), gpoolBias.data(), cx.n);
    addNCBias(regularOut.data(), gpoolBias.data(), cx.n, cx.S, regularConv.outC);
    midBN.apply(regularOut.data(), regularScratch.data(), cx.mask, rows);
    finalConv.apply(regularScratch.data(), trunk, cx.n, cx.X, cx.Y, true);
  }
};

// neuralnet/eigenbackend.cpp:1254-1303 NestedBottleneckResidualBlock
struct NestedBlock final : Block {
  BN preBN; Conv preConv; vector<std::unique_ptr<Block>> blocks; BN postBN; Conv postConv;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_BLOCK_NESTED, 1, "BLOCK_NESTED");
    int numInner = r.ints[0];
    if(numInner < 1) throw Fail("nested block: numInner must be positive");
    preBN.load(rd); preConv.load(rd);
    for(int i = 0; i < numInner; i++) {
      blocks.push_back(loadBlock(rd));
      if(blocks.back()->channels() != preConv.outC) throw Fail("nested block: inner block channel mismatch");
    }
    postBN.load(rd); postConv.load(rd);
    if(preBN.C != preConv.inC || postBN.C != preConv.outC || postConv.inC != postBN.C || postConv.outC != preBN.C)
      throw Fail("nested block: channel mismatch");
  }
  int channels() const override { return preBN.C; }
  void apply(const Ctx& cx, float* trunk) const override {
    const size_t rows = cx.rows();
    vector<float> scratch(rows * preBN.C), mid(rows * preConv.outC), midScratch(rows * preConv.outC);
    preBN.apply(trunk, scratch.data(), cx.mask, rows);
    preConv.apply(scratch.data(), mid.data(), cx.n, cx.X, cx.Y, false);
    for(auto& b : blocks) b->apply(cx, mid.data());
    postBN.apply(mid.data(), midScratch.data(), cx.mask, rows);
    postConv.apply(midScratch.data(), trunk, cx.n, cx.X, cx.Y, true);
  }
};

// neuralnet/eigenbackend.cpp:1307-1588 TransformerAttentionBlock;
// RoPE tables: neuralnet/desc.cpp:1212-1275 computeRopeCosSin.
struct AttnBlock final : Block {
  int H = 0, Hkv = 0, dq = 0, dv = 0, useRope = 0, learnable = 0;
  float theta = 0.0f;
  vector<float> freqs;
  TRMSNorm preLN; MatMul q, k, v, o;
  mutable vector<float> cosT, sinT;
  mutable int tabX = -1, tabY = -1;
  // Optional learned relative-position bias (KB_TAG_ATTNBIAS, an extension the reference's files cannot carry):
  // score(q,k) += relBias[h][yk-yq+relY-1][xk-xq+relX-1].
  vector<float> relBias;
  int relY = 0, relX = 0;

  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_BLOCK_ATTN, 6, "BLOCK_ATTN");
    H = r.ints[0]; Hkv = r.ints[1]; dq = r.ints[2]; dv = r.ints[3]; useRope = r.ints[4]; learnable = r.ints[5];
    if(H < 1 || Hkv < 1 || (H % Hkv) != 0 || dq < 1 || dv < 1) throw Fail("attention block: bad head configuration");
    if(useRope && (dq % 2) != 0) throw Fail("attention block: qHeadDim must be even with RoPE");
    if(useRope && learnable) {
      if(r.nFloats != (uint32_t)(Hkv * (dq / 2) * 2)) throw Fail("attention block: wrong number of rope freqs");
      freqs.assign(r.floats, r.floats + r.nFloats);
    } else if(useRope) {
      if(r.nFloats != 1) throw Fail("attention block: expected rope theta");
      theta = r.floats[0];
    }
    preLN.load(rd); q.load(rd); k.load(rd); v.load(rd); o.load(rd);
    if(q.inC != preLN.C || k.inC != preLN.C || v.inC != preLN.C || q.outC != H * dq || k.outC != Hkv * dq ||
       v.outC != Hkv * dv || o.inC != H * dv || o.outC != preLN.C)
      throw Fail("attention block: projection shape mismatch");
    if(!rd.atEnd() && rd.peekTag() == KB_TAG_ATTNBIAS) {
      Record rb = rd.expect(KB_TAG_ATTNBIAS, 3, "ATTNBIAS");
      relY = rb.ints[1]; relX = rb.ints[2];
      if(rb.ints[0] != H || relY < 1 || relX < 1 || rb.nFloats != (uint32_t)(H * (2 * relY - 1) * (2 * relX - 1)))
        throw Fail("attention block: relative-position bias has the wrong shape");
      relBias.assign(rb.floats, rb.floats + rb.nFloats);
    }
  }
  int channels() const override { return preLN.C; }

  void buildTables(int X, int Y) const {
    if(tabX == X && tabY == Y) return;
    const int S = X * Y, numPairs = dq / 2;
    if(learnable) {
      cosT.assign((size_t)Hkv * numPairs * S, 0.0f); sinT.assign((size_t)Hkv * numPairs * S, 0.0f);
      for(int h = 0; h < Hkv; h++)
        for(int p = 0; p < numPairs; p++) {
          float fx = freqs[(h * numPairs + p) * 2 + 0], fy = freqs[(h * numPairs + p) * 2 + 1];
          for(int y = 0; y < Y; y++)
            for(int x = 0; x < X; x++) {
              float angle = (float)x * fx + (float)y * fy;
              size_t idx = (size_t)(h * numPairs + p) * S + y * X + x;
              cosT[idx] = cosf(angle); sinT[idx] = sinf(angle);
            }
        }
    } else {
      const int numPairsPerDim = numPairs / 2, dimHalf = dq / 2;
      cosT.assign((size_t)numPairs * S, 0.0f); sinT.assign((size_t)numPairs * S, 0.0f);
      for(int p = 0; p < numPairs; p++)
        for(int y = 0; y < Y; y++)
          for(int x = 0; x < X; x++) {
            float angle;
            if(p < numPairsPerDim) {
              float freq = 1.0f / powf(theta, (float)(2 * p) / (float)dimHalf);
              angle = (float)y * freq;
            } else {
              float freq = 1.0f / powf(theta, (float)(2 * (p - numPairsPerDim)) / (float)dimHalf);
              angle = (float)x * freq;
            }
            size_t idx = (size_t)p * S + y * X + x;
            cosT[idx] = cosf(angle); sinT[idx] = sinf(angle);
          }
    }
    tabX = X; tabY = Y;
  }

  void rope(float* data, int numBufHeads, const Ctx& cx) const {
    const int numPairs = dq / 2, S = cx.S, total = numBufHeads * dq;
#pragma omp parallel for schedule(static)
    for(int b = 0; b < cx.n; b++)
      for(int xy = 0; xy < S; xy++) {
        float* row = data + ((size_t)b * S + xy) * total;
        for(int h = 0; h < numBufHeads; h++)
          for(int p = 0; p < numPairs; p++) {
            size_t t;
            if(learnable) { int kvh = h * Hkv / numBufHeads; t = (size_t)(kvh * numPairs + p) * S + xy; }
            else t = (size_t)p * S + xy;
            float c = cosT[t], s = sinT[t];
            float x0 = row[h * dq + 2 * p], x1 = row[h * dq + 2 * p + 1];
            row[h * dq + 2 * p] = x0 * c - x1 * s;
            row[h * dq + 2 * p + 1] = x0 * s + x1 * c;
          }
      }
  }

  void apply(const Ctx& cx, float* trunk) const override {
    const size_t rows = cx.rows();
    const int C = preLN.C, S = cx.S;
    vector<float> normed(rows * C), Q(rows * q.outC), K(rows * k.outC), V(rows * v.outC), A(rows * (size_t)(H * dv)), proj(rows * C);
    preLN.apply(trunk, normed.data(), cx.mask, rows);
    q.apply(normed.data(), Q.data(), rows);
    k.apply(normed.data(), K.data(), rows);
    v.apply(normed.data(), V.data(), rows);
    if(useRope) {
#pragma omp critical(ko_rope_tables)
      buildTables(cx.X, cx.Y);
      rope(Q.data(), H, cx);
      rope(K.data(), Hkv, cx);
    }
    const float scale = 1.0f / sqrtf((float)dq);
    const int group = H / Hkv;
    if(!relBias.empty() && (cx.X > relX || cx.Y > relY)) throw Fail("attention block: board larger than the relative-position bias table");
#pragma omp parallel for collapse(2) schedule(dynamic)
    for(int b = 0; b < cx.n; b++)
      for(int h = 0; h < H; h++) {
        const int kvh = h / group;
        const float* maskN = cx.mask + (size_t)b * S;
        vector<float> sc(S);
        for(int qi = 0; qi < S; qi++) {
          float* outRow = A.data() + ((size_t)b * S + qi) * (H * dv) + h * dv;
          for(int d = 0; d < dv; d++) outRow[d] = 0.0f;
          if(maskN[qi] == 0.0f) continue;  // masked query rows produce zeros (eigenbackend.cpp:1506-1511)
          const float* qv = Q.data() + ((size_t)b * S + qi) * q.outC + h * dq;
          float maxVal = -1e30f;
          for(int ki = 0; ki < S; ki++) {
            if(maskN[ki] == 0.0f) continue;
            const float* kv = K.data() + ((size_t)b * S + ki) * k.outC + kvh * dq;
            float dot = 0.0f;
            for(int d = 0; d < dq; d++) dot += qv[d] * kv[d];
            sc[ki] = dot * scale;
            if(!relBias.empty()) {
              const int dy = ki / cx.X - qi / cx.X + relY - 1, dx = ki % cx.X - qi % cx.X + relX - 1;
              sc[ki] += relBias[((size_t)h * (2 * relY - 1) + dy) * (2 * relX - 1) + dx];
            }
            maxVal = std::max(maxVal, sc[ki]);
          }
          float sumExp = 0.0f;
          for(int ki = 0; ki < S; ki++) {
            if(maskN[ki] != 0.0f) { sc[ki] = expf(sc[ki] - maxVal); sumExp += sc[ki]; }
            else sc[ki] = 0.0f;
          }
          float invSum = 1.0f / sumExp;
          for(int ki = 0; ki < S; ki++) {
            float wgt = sc[ki] * invSum;
            if(wgt == 0.0f) continue;
            const float* vv = V.data() + ((size_t)b * S + ki) * v.outC + kvh * dv;
            for(int d = 0; d < dv; d++) outRow[d] += wgt * vv[d];
          }
        }
      }
    o.apply(A.data(), proj.data(), rows);
#pragma omp parallel for schedule(static)
    for(size_t r = 0; r < rows; r++) {
      float mv = cx.mask[r];
      for(int c = 0; c < C; c++) trunk[r * C + c] += proj[r * C + c] * mv;
    }
  }
};

// neuralnet/eigenbackend.cpp:1592-1707 TransformerFFNBlock
struct FFNBlock final : Block {
  int C = 0, ffnC = 0, swiglu = 0;
  TRMSNorm preLN; MatMul l1, gate, l2;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_BLOCK_FFN, 3, "BLOCK_FFN");
    C = r.ints[0]; ffnC = r.ints[1]; swiglu = r.ints[2];
    // The Eigen backend throws for non-SwiGLU FFN blocks (eigenbackend.cpp:1621-1623).
    if(!swiglu) throw Fail("ffn block: non-SwiGLU FFN is not supported");
    preLN.load(rd); l1.load(rd); gate.load(rd); l2.load(rd);
    if(preLN.C != C || l1.inC != C || l1.outC != ffnC || gate.inC != C || gate.outC != ffnC || l2.inC != ffnC || l2.outC != C)
      throw Fail("ffn block: shape mismatch");
  }
  int channels() const override { return C; }
  void apply(const Ctx& cx, float* trunk) const override {
    const size_t rows = cx.rows();
    vector<float> normed(rows * C), a(rows * ffnC), g(rows * ffnC), proj(rows * C);
    preLN.apply(trunk, normed.data(), cx.mask, rows);
    l1.apply(normed.data(), a.data(), rows);
    gate.apply(normed.data(), g.data(), rows);
#pragma omp parallel for schedule(static)
    for(size_t i = 0; i < rows * (size_t)ffnC; i++) {
      float x = a[i];
      a[i] = (x / (1.0f + expf(-x))) * g[i];
    }
    l2.apply(a.data(), proj.data(), rows);
#pragma omp parallel for schedule(static)
    for(size_t r = 0; r < rows; r++) {
      float mv = cx.mask[r];
      for(int c = 0; c < C; c++) trunk[r * C + c] += proj[r * C + c] * mv;
    }
  }
};

std::unique_ptr<Block> loadBlock(Reader& rd) {
  switch(rd.peekTag()) {
    case KB_TAG_BLOCK_ORDINARY: { auto b = std::make_unique<OrdinaryBlock>(); b->load(rd); return b; }
    case KB_TAG_BLOCK_GPOOL: { auto b = std::make_unique<GPoolBlock>(); b->load(rd); return b; }
    case KB_TAG_BLOCK_NESTED: { auto b = std::make_unique<NestedBlock>(); b->load(rd); return b; }
    case KB_TAG_BLOCK_ATTN: { auto b = std::make_unique<AttnBlock>(); b->load(rd); return b; }
    case KB_TAG_BLOCK_FFN: { auto b = std::make_unique<FFNBlock>(); b->load(rd); return b; }
    default: throw Fail("unknown block tag " + std::to_string(rd.peekTag()));
  }
}

// ------------------------------------------------------------------------------------------------
// Trunk and heads

// neuralnet/eigenbackend.cpp:1851-1936
struct Trunk {
  int numBlocks = 0, trunkC = 0, normKind = 0;
  Conv initialConv; MatMul initialMatMul;
  // SGF metadata encoder, neuralnet/eigenbackend.cpp:1801-1847 (parsed by desc.cpp:1476-1522); inMetaC == 0: absent
  int inMetaC = 0, metaAct1 = 0, metaAct2 = 0;
  MatMul metaMul1, metaMul2, metaMul3; MatBias metaBias1, metaBias2;
  vector<std::unique_ptr<Block>> blocks;
  BN tipBN; RMSNorm tipRMS;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_TRUNK, 6, "TRUNK");
    numBlocks = r.ints[0]; trunkC = r.ints[1]; normKind = r.ints[5];
    if(numBlocks < 1) throw Fail("trunk: numBlocks must be positive");
    initialConv.load(rd); initialMatMul.load(rd);
    if(initialConv.outC != trunkC || initialMatMul.outC != trunkC) throw Fail("trunk: initial layer channel mismatch");
    if(inMetaC > 0) {
      Record e = rd.expect(KB_TAG_METAENC, 2, "METAENC");
      if(e.ints[1] != inMetaC) throw Fail("metadata encoder: channel count differs from the model record");
      metaMul1.load(rd); metaBias1.load(rd); metaAct1 = loadAct(rd);
      metaMul2.load(rd); metaBias2.load(rd); metaAct2 = loadAct(rd);
      metaMul3.load(rd);
      if(metaMul1.inC != inMetaC || metaMul1.outC != metaBias1.C || metaMul2.inC != metaMul1.outC || metaMul2.outC != metaBias2.C ||
         metaMul3.inC != metaMul2.outC || metaMul3.outC != trunkC)
        throw Fail("metadata encoder: shape mismatch");
    }
    for(int i = 0; i < numBlocks; i++) {
      blocks.push_back(loadBlock(rd));
      if(blocks.back()->channels() != trunkC) throw Fail("trunk: block channel mismatch");
    }
    if(normKind == 0) { tipBN.load(rd); if(tipBN.C != trunkC) throw Fail("trunk: tip BN channel mismatch"); }
    else if(normKind == 1) { tipRMS.load(rd); if(tipRMS.C != trunkC) throw Fail("trunk: tip RMSNorm channel mismatch"); }
    else throw Fail("trunk: unknown norm kind");
  }
  // streams (optional): [numBlocks + 1][rows][trunkC], the residual stream entering each block and leaving the last
  void apply(const Ctx& cx, const float* input, const float* global, const float* meta, float* trunkOut, float* streams = nullptr) const {
    const size_t rows = cx.rows();
    vector<float> t(rows * trunkC), gbias((size_t)cx.n * trunkC);
    initialConv.apply(input, t.data(), cx.n, cx.X, cx.Y, false);
    initialMatMul.apply(global, gbias.data(), cx.n);
    addNCBias(t.data(), gbias.data(), cx.n, cx.S, trunkC);
    if(inMetaC > 0) {
      // eigenbackend.cpp:1917-1920: the encoder's output is a second per-sample bias on the trunk
      vector<float> h1((size_t)cx.n * metaMul1.outC), h2((size_t)cx.n * metaMul2.outC);
      metaMul1.apply(meta, h1.data(), cx.n);
      metaBias1.apply(h1.data(), cx.n);
      for(float& x : h1) x = applyAct(x, metaAct1);
      metaMul2.apply(h1.data(), h2.data(), cx.n);
      metaBias2.apply(h2.data(), cx.n);
      for(float& x : h2) x = applyAct(x, metaAct2);
      metaMul3.apply(h2.data(), gbias.data(), cx.n);
      addNCBias(t.data(), gbias.data(), cx.n, cx.S, trunkC);
    }
    for(size_t i = 0; i < blocks.size(); i++) {
      if(streams) std::memcpy(streams + i * t.size(), t.data(), t.size() * sizeof(float));
      blocks[i]->apply(cx, t.data());
    }
    if(streams) std::memcpy(streams + blocks.size() * t.size(), t.data(), t.size() * sizeof(float));
    if(!trunkOut) return;
    if(normKind == 0) tipBN.apply(t.data(), trunkOut, cx.mask, rows);
    else tipRMS.apply(t.data(), trunkOut, cx.mask, cx.n, cx.S);
  }
};

// neuralnet/eigenbackend.cpp:1938-2025
struct PolicyHead {
  int modelVersion = 0, policyC = 0, hasPassMlp = 0;
  Conv p1Conv, g1Conv; BN g1BN; MatMul gpoolToBias; BN p1BN; Conv p2Conv; MatMul passMul; MatBias passBias; int passAct = 0; MatMul passMul2;
  void load(Reader& rd) {
    Record r = rd.expect(KB_TAG_POLICYHEAD, 3, "POLICYHEAD");
    modelVersion = r.ints[0]; policyC = r.ints[1]; hasPassMlp = r.ints[2];
    p1Conv.load(rd); g1Conv.load(rd); g1BN.load(rd); gpoolToBias.load(rd); p1BN.load(rd); p2Conv.load(rd); passMul.load(rd);
    if(hasPassMlp) { passBias.load(rd); passAct = loadAct(rd); passMul2.load(rd); }
    if(p1Conv.outC != p1BN.C || g1Conv.outC != g1BN.C || gpoolToBias.inC != 3 * g1BN.C || gpoolToBias.outC != p1BN.C ||
       p2Conv.inC != p1BN.C || p2Conv.outC != policyC || passMul.inC != 3 * g1BN.C)
      throw Fail("policy head: shape mismatch");
    if(hasPassMlp ? (passMul.outC != passBias.C || passMul2.inC != passMul.outC || passMul2.outC != policyC) : (passMul.outC != policyC))
      throw Fail("policy head: pass shape mismatch");
  }
  void apply(const Ctx& cx, const float* trunk, float* policy, float* policyPass) const {
    const size_t rows = cx.rows();
    vector<float> p1(rows * p1Conv.outC), p1b(rows * p1Conv.outC), g1(rows * g1Conv.outC), g1b(rows * g1Conv.outC);
    vector<float> concat((size_t)cx.n * 3 * g1Conv.outC), bias((size_t)cx.n * p1Conv.outC);
    p1Conv.apply(trunk, p1.data(), cx.n, cx.X, cx.Y, false);
    g1Conv.apply(trunk, g1.data(), cx.n, cx.X, cx.Y, false);
    g1BN.apply(g1.data(), g1b.data(), cx.mask, rows);
    if(emuOn(KO_EMU_CONV_INPUTS)) { roundTensor(g1b.data(), g1b.size()); roundTensor(p1.data(), p1.size()); }
    poolRowsGPool(g1b.data(), concat.data(), cx.mask, cx.maskSum, cx.n, cx.S, g1Conv.outC);
    gpoolToBias.apply(concat.data(), bias.data(), cx.n);
    addNCBias(p1.data(), bias.data(), cx.n, cx.S, p1Conv.outC);
    p1BN.apply(p1.data(), p1b.data(), cx.mask, rows);
    p2Conv.apply(p1b.data(), policy, cx.n, cx.X, cx.Y, false);
    if(hasPassMlp) {
      vector<float> pass((size_t)cx.n * passMul.outC);
      passMul.apply(concat.data(), pass.data(), cx.n);
      passBias.apply(pass.data(), cx.n);
      for(float& x : pass) x = applyAct(x, passAct);
      passMul2.apply(pass.data(), policyPass, cx.n);
    } else {
      passMul.apply(concat.data(), policyPass, cx.n);
    }
  }
};

// neuralnet/eigenbackend.cpp:2027-2103
struct ValueHead {
  Conv v1Conv; BN v1BN; MatMul v2Mul; MatBias v2Bias; int v2Act = 0; MatMul v3Mul; MatBias v3Bias; MatMul sv3Mul; MatBias sv3Bias; Conv ownConv;
  void load(Reader& rd) {
    rd.expect(KB_TAG_VALUEHEAD, 1, "VALUEHEAD");
    v1Conv.load(rd); v1BN.load(rd); v2Mul.load(rd); v2Bias.load(rd); v2Act = loadAct(rd);
    v3Mul.load(rd); v3Bias.load(rd); sv3Mul.load(rd); sv3Bias.load(rd); ownConv.load(rd);
    if(v1Conv.outC != v1BN.C || v2Mul.inC != 3 * v1BN.C || v2Mul.outC != v2Bias.C || v3Mul.inC != v2Mul.outC ||
       v3Mul.outC != v3Bias.C || sv3Mul.inC != v2Mul.outC || sv3Mul.outC != sv3Bias.C || ownConv.inC != v1BN.C)
      throw Fail("value head: shape mismatch");
  }
  void apply(const Ctx& cx, const float* trunk, float* value, float* scoreValue, float* ownership) const {
    const size_t rows = cx.rows();
    vector<float> v1(rows * v1Conv.outC), v1b(rows * v1Conv.outC), mean((size_t)cx.n * 3 * v1Conv.outC), v2((size_t)cx.n * v2Mul.outC);
    v1Conv.apply(trunk, v1.data(), cx.n, cx.X, cx.Y, false);
    v1BN.apply(v1.data(), v1b.data(), cx.mask, rows);
    if(emuOn(KO_EMU_CONV_INPUTS)) roundTensor(v1b.data(), v1b.size());
    poolRowsValueHead(v1b.data(), mean.data(), cx.maskSum, cx.n, cx.S, v1Conv.outC);
    v2Mul.apply(mean.data(), v2.data(), cx.n);
    v2Bias.apply(v2.data(), cx.n);
    for(float& x : v2) x = applyAct(x, v2Act);
    v3Mul.apply(v2.data(), value, cx.n);
    v3Bias.apply(value, cx.n);
    sv3Mul.apply(v2.data(), scoreValue, cx.n);
    sv3Bias.apply(scoreValue, cx.n);
    ownConv.apply(v1b.data(), ownership, cx.n, cx.X, cx.Y, false);
  }
};

}  // namespace

struct ko_model {
  int X = 0, Y = 0;
  int modelVersion = 0, inC = 0, inGlobalC = 0, inMetaC = 0, policyC = 0, valueC = 0, scoreValueC = 0, ownershipC = 0;
  Trunk trunk; PolicyHead policyHead; ValueHead valueHead;
};

namespace {
template <class F>
int guarded(F&& f) {
  try { f(); return 0; }
  catch(const std::exception& e) { g_lastError = e.what(); return 1; }
  catch(...) { g_lastError = "unknown error"; return 2; }
}
}  // namespace

extern "C" {

const char* ko_last_error(void) { return g_lastError.c_str(); }

int ko_set_storage_emulation(int storageType, int flags) {
  if(storageType < 0 || storageType > 2) return 1;
  g_emuType = storageType;
  g_emuFlags = flags;
  return 0;
}

int ko_set_num_threads(int n) {
#ifdef _OPENMP
  if(n < 1) return 1;
  omp_set_num_threads(n);
  return 0;
#else
  return n == 1 ? 0 : 1;
#endif
}

int ko_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

int ko_model_create(const void* blob, size_t nbytes, int nnXLen, int nnYLen, ko_model** out) {
  if(out) *out = nullptr;
  return guarded([&]() {
    if(out == nullptr) throw Fail("ko_model_create: out is NULL");
    if(nnXLen < 2 || nnYLen < 2 || nnXLen > 50 || nnYLen > 50) throw Fail("ko_model_create: board size out of range");
    Reader rd(blob, nbytes);
    auto m = std::make_unique<ko_model>();
    m->X = nnXLen; m->Y = nnYLen;
    Record r = rd.expect(KB_TAG_MODEL, 8, "MODEL");
    m->modelVersion = r.ints[0]; m->inC = r.ints[1]; m->inGlobalC = r.ints[2]; m->inMetaC = r.ints[3];
    m->policyC = r.ints[4]; m->valueC = r.ints[5]; m->scoreValueC = r.ints[6]; m->ownershipC = r.ints[7];
    if(m->inMetaC < 0) throw Fail("model: bad metadata channel count");
    m->trunk.inMetaC = m->inMetaC;
    m->trunk.load(rd); m->policyHead.load(rd); m->valueHead.load(rd);
    rd.expect(KB_TAG_END, 0, "END");
    if(m->trunk.initialConv.inC != m->inC || m->trunk.initialMatMul.inC != m->inGlobalC) throw Fail("model: input channel mismatch");
    if(m->policyHead.policyC != m->policyC || m->valueHead.v3Mul.outC != m->valueC ||
       m->valueHead.sv3Mul.outC != m->scoreValueC || m->valueHead.ownConv.outC != m->ownershipC || m->ownershipC != 1)
      throw Fail("model: output channel mismatch");
    if(m->policyHead.p1Conv.inC != m->trunk.trunkC || m->valueHead.v1Conv.inC != m->trunk.trunkC) throw Fail("model: head input mismatch");
    *out = m.release();
  });
}

void ko_model_destroy(ko_model* m) { delete m; }

int ko_model_info(const ko_model* m, int32_t info[9]) {
  return guarded([&]() {
    if(!m || !info) throw Fail("ko_model_info: NULL argument");
    info[0] = m->modelVersion; info[1] = m->inC; info[2] = m->inGlobalC; info[3] = m->policyC; info[4] = m->valueC;
    info[5] = m->scoreValueC; info[6] = m->ownershipC; info[7] = m->trunk.trunkC; info[8] = m->trunk.numBlocks;
  });
}

int ko_model_meta_channels(const ko_model* m, int32_t* channels) {
  return guarded([&]() {
    if(!m || !channels) throw Fail("ko_model_meta_channels: NULL argument");
    *channels = m->inMetaC;
  });
}

int ko_forward(
  const ko_model* m, int n, const float* spatial, const float* global,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership, float* trunkOut) {
  return ko_forward_meta(m, n, spatial, global, nullptr, policy, policyPass, value, scoreValue, ownership, trunkOut);
}

int ko_forward_meta(
  const ko_model* m, int n, const float* spatial, const float* global, const float* meta,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership, float* trunkOut) {
  return guarded([&]() {
    if(!m || !spatial || !global) throw Fail("ko_forward: NULL argument");
    if(n < 1) throw Fail("ko_forward: batch size must be positive");
    if((m->inMetaC > 0) != (meta != nullptr)) throw Fail("ko_forward: metadata rows must be given exactly for models with a metadata encoder");
    const int S = m->X * m->Y;
    const size_t rows = (size_t)n * S;
    // mask = input channel 0, maskSum = its per-sample sum (eigenbackend.cpp:2169-2170, 122-133)
    vector<float> mask(rows), maskSum(n);
    for(size_t r = 0; r < rows; r++) mask[r] = spatial[r * m->inC];
    for(int b = 0; b < n; b++) {
      float s = 0.0f;
      for(int p = 0; p < S; p++) s += mask[(size_t)b * S + p];
      maskSum[b] = s;
    }
    Ctx cx{n, m->X, m->Y, S, mask.data(), maskSum.data()};
    vector<float> trunkBuf(rows * m->trunk.trunkC);
    m->trunk.apply(cx, spatial, global, meta, trunkBuf.data());
    if(trunkOut) std::memcpy(trunkOut, trunkBuf.data(), trunkBuf.size() * sizeof(float));
    vector<float> pol(rows * m->policyC), pass((size_t)n * m->policyC), val((size_t)n * m->valueC), sv((size_t)n * m->scoreValueC), own(rows);
    m->policyHead.apply(cx, trunkBuf.data(), pol.data(), pass.data());
    m->valueHead.apply(cx, trunkBuf.data(), val.data(), sv.data(), own.data());
    if(policy) std::memcpy(policy, pol.data(), pol.size() * sizeof(float));
    if(policyPass) std::memcpy(policyPass, pass.data(), pass.size() * sizeof(float));
    if(value) std::memcpy(value, val.data(), val.size() * sizeof(float));
    if(scoreValue) std::memcpy(scoreValue, sv.data(), sv.size() * sizeof(float));
    if(ownership) std::memcpy(ownership, own.data(), own.size() * sizeof(float));
  });
}

int ko_trunk_streams(const ko_model* m, int n, const float* spatial, const float* global, const float* meta, float* streams) {
  return guarded([&]() {
    if(!m || !spatial || !global || !streams) throw Fail("ko_trunk_streams: NULL argument");
    if(n < 1) throw Fail("ko_trunk_streams: batch size must be positive");
    if((m->inMetaC > 0) != (meta != nullptr)) throw Fail("ko_trunk_streams: metadata rows must be given exactly for models with a metadata encoder");
    const int S = m->X * m->Y;
    const size_t rows = (size_t)n * S;
    vector<float> mask(rows), maskSum(n);
    for(size_t r = 0; r < rows; r++) mask[r] = spatial[r * m->inC];
    for(int b = 0; b < n; b++) {
      float s = 0.0f;
      for(int p = 0; p < S; p++) s += mask[(size_t)b * S + p];
      maskSum[b] = s;
    }
    Ctx cx{n, m->X, m->Y, S, mask.data(), maskSum.data()};
    m->trunk.apply(cx, spatial, global, meta, nullptr, streams);
  });
}

int ko_eval_layer(
  const void* blob, size_t nbytes, int n, int nnXLen, int nnYLen, const float* in, const float* mask, float* out) {
  return guarded([&]() {
    if(!in || !out) throw Fail("ko_eval_layer: NULL argument");
    if(n < 1 || nnXLen < 1 || nnYLen < 1) throw Fail("ko_eval_layer: bad sizes");
    Reader rd(blob, nbytes);
    const int S = nnXLen * nnYLen;
    const size_t rows = (size_t)n * S;
    uint32_t tag = rd.peekTag();
    if(tag == KB_TAG_CONV) {
      Conv c; c.load(rd);
      c.apply(in, out, n, nnXLen, nnYLen, false);
      return;
    }
    if(!mask) throw Fail("ko_eval_layer: mask required");
    vector<float> maskSum(n);
    for(int b = 0; b < n; b++) {
      float s = 0.0f;
      for(int p = 0; p < S; p++) s += mask[(size_t)b * S + p];
      maskSum[b] = s;
    }
    Ctx cx{n, nnXLen, nnYLen, S, mask, maskSum.data()};
    if(tag == KB_TAG_BN) {
      BN b; b.load(rd);
      b.apply(in, out, mask, rows);
    } else if(tag == KB_TAG_BLOCK_ORDINARY || tag == KB_TAG_BLOCK_GPOOL || tag == KB_TAG_BLOCK_NESTED ||
              tag == KB_TAG_BLOCK_ATTN || tag == KB_TAG_BLOCK_FFN) {
      auto b = loadBlock(rd);
      std::memcpy(out, in, rows * b->channels() * sizeof(float));
      b->apply(cx, out);
    } else {
      throw Fail("ko_eval_layer: unsupported layer tag " + std::to_string(tag));
    }
  });
}

}  // extern "C"
