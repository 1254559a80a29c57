// Host-side network description parsed from a model blob (include/kb_modelblob.h).
// Plain data: weights stay fp32 in the reference's index order (cpp/neuralnet/desc.h) until a
// handle repacks them for the device.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "../../include/kb_modelblob.h"

namespace kb {

struct ConvW {
  int kY = 0, kX = 0, inC = 0, outC = 0;
  std::vector<float> w;  // [oc][ic][y][x]
};
struct BNW {
  int C = 0, act = 0;
  std::vector<float> scale, bias;  // merged (desc.cpp:278-285)
};
struct MatMulW {
  int inC = 0, outC = 0;
  std::vector<float> w;  // [ic][oc]
};
struct MatBiasW {
  int C = 0;
  std::vector<float> b;
};
struct TRMSNormW {
  int C = 0;
  float eps = 0.0f;
  std::vector<float> weight;
};
struct RMSNormW {
  int C = 0, spatial = 0, act = 0;
  float eps = 0.0f;
  std::vector<float> gamma, beta;
};

enum BlockKind { BLOCK_ORDINARY = 0, BLOCK_GPOOL = 1, BLOCK_NESTED = 2, BLOCK_ATTN = 3, BLOCK_FFN = 4 };

// One residual block of any kind; unused members stay empty.
struct BlockW {
  int kind = BLOCK_ORDINARY;
  // ordinary: preBN conv1 midBN conv2.   gpool: preBN conv1(regular) gpoolConv gpoolBN gpoolToBias midBN conv2(final).
  // nested:   preBN conv1(pre 1x1) inner* midBN(post BN) conv2(post 1x1).
  BNW preBN, midBN, gpoolBN;
  ConvW conv1, conv2, gpoolConv;
  MatMulW gpoolToBias;
  std::vector<BlockW> inner;
  // attention (eigenbackend.cpp:1307-1588)
  int heads = 0, kvHeads = 0, qDim = 0, vDim = 0, useRope = 0, learnableRope = 0;
  float ropeTheta = 0.0f;
  std::vector<float> ropeFreqs;
  // optional relative-position bias [heads][2*relBiasY-1][2*relBiasX-1] (empty: none)
  std::vector<float> relBias;
  int relBiasY = 0, relBiasX = 0;
  TRMSNormW preLN;
  MatMulW q, k, v, out;
  // ffn (eigenbackend.cpp:1592-1707)
  int ffnC = 0;
  MatMulW linear1, gate, linear2;

  int channels() const { return (kind == BLOCK_ATTN || kind == BLOCK_FFN) ? preLN.C : preBN.C; }
};

struct Model {
  int modelVersion = 0, inC = 0, inGlobalC = 0, inMetaC = 0, policyC = 0, valueC = 0, scoreValueC = 0, ownershipC = 0;
  // trunk
  int numBlocks = 0, trunkC = 0, normKind = 0;
  ConvW initialConv;
  MatMulW initialMatMul;
  // SGF metadata encoder (only if inMetaC > 0): mul1 bias1 act1 mul2 bias2 act2 mul3 -> [n][trunkC] (eigenbackend.cpp:1801-1847)
  int metaEncoderVersion = 0, metaAct1 = 0, metaAct2 = 0;
  MatMulW metaMul1, metaMul2, metaMul3;
  MatBiasW metaBias1, metaBias2;
  std::vector<BlockW> blocks;
  BNW tipBN;
  RMSNormW tipRMS;
  // policy head (eigenbackend.cpp:1938-2025)
  int hasPassMlp = 0, passAct = 0;
  ConvW p1Conv, g1Conv, p2Conv;
  BNW g1BN, p1BN;
  MatMulW gpoolToBias, passMul, passMul2;
  MatBiasW passBias;
  // value head (eigenbackend.cpp:2027-2103)
  int v2Act = 0;
  ConvW v1Conv, ownConv;
  BNW v1BN;
  MatMulW v2Mul, v3Mul, sv3Mul;
  MatBiasW v2Bias, v3Bias, sv3Bias;
};

// Throws std::runtime_error on malformed or inconsistent input.
void parseModel(const void* blob, size_t nbytes, Model& out);

// Single-layer parsers for kb_eval_layer.
void parseConv(kbblob::Reader& rd, ConvW& out);
void parseBN(kbblob::Reader& rd, BNW& out);
void parseBlock(kbblob::Reader& rd, BlockW& out);

}  // namespace kb
