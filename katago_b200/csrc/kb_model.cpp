// Model blob -> kb::Model.  Validates every shape relation the reference's loader enforces
// (cpp/neuralnet/desc.cpp:557-568, 640-670, 765-776, 1129-1136, 1306-1317, 1971-2017, 2128-2188,
// 2412-2442) so that a malformed blob fails here, on the host, before any launch.
#include "kb_model.h"

#include <stdexcept>

namespace kb {

using kbblob::Reader;
using kbblob::Record;

static void fail(const std::string& msg) { throw std::runtime_error("model: " + msg); }

void parseConv(Reader& rd, ConvW& c) {
  Record r = rd.expect(KB_TAG_CONV, 6, "CONV");
  c.kY = r.ints[0]; c.kX = r.ints[1]; c.inC = r.ints[2]; c.outC = r.ints[3];
  if(c.kY <= 0 || c.kX <= 0 || (c.kY % 2) != 1 || (c.kX % 2) != 1) fail("convolution sizes must be odd and positive");
  if(c.kY > 7 || c.kX > 7) fail("convolution sizes above 7 are not supported");
  if(c.inC <= 0 || c.outC <= 0) fail("convolution channels must be positive");
  if(r.ints[4] != 1 || r.ints[5] != 1) fail("dilated convolutions are not supported");
  if((size_t)r.nFloats != (size_t)c.kY * c.kX * c.inC * c.outC) fail("convolution has the wrong number of weights");
  c.w.assign(r.floats, r.floats + r.nFloats);
}

void parseBN(Reader& rd, BNW& b) {
  Record r = rd.expect(KB_TAG_BN, 2, "BN");
  b.C = r.ints[0]; b.act = r.ints[1];
  if(b.C <= 0 || r.nFloats != (uint32_t)(2 * b.C)) fail("batch norm has the wrong number of values");
  if(b.act != KB_ACT_IDENTITY && b.act != KB_ACT_RELU && b.act != KB_ACT_MISH && b.act != KB_ACT_SILU && b.act != KB_ACT_MISH_SCALE8)
    fail("unknown activation");
  b.scale.assign(r.floats, r.floats + b.C);
  b.bias.assign(r.floats + b.C, r.floats + 2 * b.C);
}

static void parseMatMul(Reader& rd, MatMulW& m) {
  Record r = rd.expect(KB_TAG_MATMUL, 2, "MATMUL");
  m.inC = r.ints[0]; m.outC = r.ints[1];
  if(m.inC <= 0 || m.outC <= 0 || (size_t)r.nFloats != (size_t)m.inC * m.outC) fail("matmul has the wrong number of weights");
  m.w.assign(r.floats, r.floats + r.nFloats);
}

static void parseMatBias(Reader& rd, MatBiasW& m) {
  Record r = rd.expect(KB_TAG_MATBIAS, 1, "MATBIAS");
  m.C = r.ints[0];
  if(m.C <= 0 || r.nFloats != (uint32_t)m.C) fail("matbias has the wrong number of values");
  m.b.assign(r.floats, r.floats + m.C);
}

static int parseAct(Reader& rd) {
  Record r = rd.expect(KB_TAG_ACT, 1, "ACT");
  return r.ints[0];
}

static void parseTRMS(Reader& rd, TRMSNormW& t) {
  Record r = rd.expect(KB_TAG_TRMSNORM, 1, "TRMSNORM");
  t.C = r.ints[0];
  if(t.C <= 0 || r.nFloats != (uint32_t)(t.C + 1)) fail("transformer rmsnorm has the wrong number of values");
  t.eps = r.floats[0];
  t.weight.assign(r.floats + 1, r.floats + 1 + t.C);
}

void parseBlock(Reader& rd, BlockW& b) {
  uint32_t tag = rd.peekTag();
  if(tag == KB_TAG_BLOCK_ORDINARY) {
    rd.next();
    b.kind = BLOCK_ORDINARY;
    parseBN(rd, b.preBN); parseConv(rd, b.conv1); parseBN(rd, b.midBN); parseConv(rd, b.conv2);
    if(b.preBN.C != b.conv1.inC || b.conv1.outC != b.midBN.C || b.midBN.C != b.conv2.inC || b.conv2.outC != b.preBN.C)
      fail("ordinary block channel mismatch");
  }
  else if(tag == KB_TAG_BLOCK_GPOOL) {
    rd.next();
    b.kind = BLOCK_GPOOL;
    parseBN(rd, b.preBN); parseConv(rd, b.conv1); parseConv(rd, b.gpoolConv); parseBN(rd, b.gpoolBN);
    parseMatMul(rd, b.gpoolToBias); parseBN(rd, b.midBN); parseConv(rd, b.conv2);
    if(b.preBN.C != b.conv1.inC || b.preBN.C != b.gpoolConv.inC || b.gpoolConv.outC != b.gpoolBN.C ||
       b.gpoolToBias.inC != 3 * b.gpoolBN.C || b.gpoolToBias.outC != b.conv1.outC || b.midBN.C != b.conv1.outC ||
       b.conv2.inC != b.midBN.C || b.conv2.outC != b.preBN.C)
      fail("gpool block channel mismatch");
  }
  else if(tag == KB_TAG_BLOCK_NESTED) {
    Record r = rd.expect(KB_TAG_BLOCK_NESTED, 1, "BLOCK_NESTED");
    b.kind = BLOCK_NESTED;
    int numInner = r.ints[0];
    if(numInner < 1 || numInner > 64) fail("nested block: bad inner block count");
    parseBN(rd, b.preBN); parseConv(rd, b.conv1);
    b.inner.resize(numInner);
    for(int i = 0; i < numInner; i++) {
      parseBlock(rd, b.inner[i]);
      if(b.inner[i].channels() != b.conv1.outC) fail("nested block: inner block channel mismatch");
    }
    parseBN(rd, b.midBN); parseConv(rd, b.conv2);
    if(b.preBN.C != b.conv1.inC || b.midBN.C != b.conv1.outC || b.conv2.inC != b.midBN.C || b.conv2.outC != b.preBN.C)
      fail("nested block channel mismatch");
  }
  else if(tag == KB_TAG_BLOCK_ATTN) {
    Record r = rd.expect(KB_TAG_BLOCK_ATTN, 6, "BLOCK_ATTN");
    b.kind = BLOCK_ATTN;
    b.heads = r.ints[0]; b.kvHeads = r.ints[1]; b.qDim = r.ints[2]; b.vDim = r.ints[3]; b.useRope = r.ints[4]; b.learnableRope = r.ints[5];
    if(b.heads < 1 || b.kvHeads < 1 || (b.heads % b.kvHeads) != 0 || b.qDim < 1 || b.vDim < 1) fail("attention block: bad head configuration");
    if(b.useRope && (b.qDim % 2) != 0) fail("attention block: qHeadDim must be even when RoPE is used");
    if(b.useRope && b.learnableRope) {
      if(r.nFloats != (uint32_t)(b.kvHeads * (b.qDim / 2) * 2)) fail("attention block: wrong number of rope frequencies");
      b.ropeFreqs.assign(r.floats, r.floats + r.nFloats);
    }
    else if(b.useRope) {
      if(r.nFloats != 1 || !(r.floats[0] > 0.0f)) fail("attention block: rope theta must be positive");
      b.ropeTheta = r.floats[0];
    }
    parseTRMS(rd, b.preLN); parseMatMul(rd, b.q); parseMatMul(rd, b.k); parseMatMul(rd, b.v); parseMatMul(rd, b.out);
    if(b.q.inC != b.preLN.C || b.k.inC != b.preLN.C || b.v.inC != b.preLN.C || b.q.outC != b.heads * b.qDim ||
       b.k.outC != b.kvHeads * b.qDim || b.v.outC != b.kvHeads * b.vDim || b.out.inC != b.heads * b.vDim || b.out.outC != b.preLN.C)
      fail("attention block: projection shape mismatch");
    if(!rd.atEnd() && rd.peekTag() == KB_TAG_ATTNBIAS) {
      Record rb = rd.expect(KB_TAG_ATTNBIAS, 3, "ATTNBIAS");
      b.relBiasY = rb.ints[1]; b.relBiasX = rb.ints[2];
      if(rb.ints[0] != b.heads || b.relBiasY < 1 || b.relBiasX < 1 || b.relBiasY > 64 || b.relBiasX > 64 ||
         rb.nFloats != (uint32_t)(b.heads * (2 * b.relBiasY - 1) * (2 * b.relBiasX - 1)))
        fail("attention block: relative-position bias has the wrong shape");
      b.relBias.assign(rb.floats, rb.floats + rb.nFloats);
    }
  }
  else if(tag == KB_TAG_BLOCK_FFN) {
    Record r = rd.expect(KB_TAG_BLOCK_FFN, 3, "BLOCK_FFN");
    b.kind = BLOCK_FFN;
    int C = r.ints[0];
    b.ffnC = r.ints[1];
    // The reference's CPU backend rejects non-SwiGLU FFN blocks (eigenbackend.cpp:1621-1623).
    if(!r.ints[2]) fail("ffn block: non-SwiGLU FFN is not supported");
    parseTRMS(rd, b.preLN); parseMatMul(rd, b.linear1); parseMatMul(rd, b.gate); parseMatMul(rd, b.linear2);
    if(b.preLN.C != C || b.linear1.inC != C || b.linear1.outC != b.ffnC || b.gate.inC != C || b.gate.outC != b.ffnC ||
       b.linear2.inC != b.ffnC || b.linear2.outC != C)
      fail("ffn block: shape mismatch");
  }
  else {
    fail("unknown block tag " + std::to_string(tag));
  }
}

void parseModel(const void* blob, size_t nbytes, Model& m) {
  Reader rd(blob, nbytes);
  Record r = rd.expect(KB_TAG_MODEL, 8, "MODEL");
  m.modelVersion = r.ints[0]; m.inC = r.ints[1]; m.inGlobalC = r.ints[2]; m.inMetaC = r.ints[3];
  m.policyC = r.ints[4]; m.valueC = r.ints[5]; m.scoreValueC = r.ints[6]; m.ownershipC = r.ints[7];
  if(m.inMetaC < 0 || m.inMetaC > 4096) fail("bad metadata channel count");
  r = rd.expect(KB_TAG_TRUNK, 6, "TRUNK");
  m.numBlocks = r.ints[0]; m.trunkC = r.ints[1]; m.normKind = r.ints[5];
  if(m.numBlocks < 1 || m.numBlocks > 4096) fail("bad trunk block count");
  parseConv(rd, m.initialConv);
  parseMatMul(rd, m.initialMatMul);
  if(m.initialConv.inC != m.inC || m.initialConv.outC != m.trunkC || m.initialMatMul.inC != m.inGlobalC || m.initialMatMul.outC != m.trunkC)
    fail("trunk initial layers do not match the declared channel counts");
  if(m.inMetaC > 0) {
    Record e = rd.expect(KB_TAG_METAENC, 2, "METAENC");
    m.metaEncoderVersion = e.ints[0];
    if(e.ints[1] != m.inMetaC) fail("metadata encoder: channel count differs from the model record");
    parseMatMul(rd, m.metaMul1); parseMatBias(rd, m.metaBias1); m.metaAct1 = parseAct(rd);
    parseMatMul(rd, m.metaMul2); parseMatBias(rd, m.metaBias2); m.metaAct2 = parseAct(rd);
    parseMatMul(rd, m.metaMul3);
    if(m.metaMul1.inC != m.inMetaC || m.metaMul1.outC != m.metaBias1.C || m.metaMul2.inC != m.metaMul1.outC ||
       m.metaMul2.outC != m.metaBias2.C || m.metaMul3.inC != m.metaMul2.outC || m.metaMul3.outC != m.trunkC)
      fail("metadata encoder shape mismatch");
  }
  m.blocks.resize(m.numBlocks);
  for(int i = 0; i < m.numBlocks; i++) {
    parseBlock(rd, m.blocks[i]);
    if(m.blocks[i].channels() != m.trunkC) fail("trunk block channel mismatch");
  }
  if(m.normKind == 0) {
    parseBN(rd, m.tipBN);
    if(m.tipBN.C != m.trunkC) fail("trunk tip norm channel mismatch");
  }
  else if(m.normKind == 1) {
    Record t = rd.expect(KB_TAG_RMSNORM, 3, "RMSNORM");
    m.tipRMS.C = t.ints[0]; m.tipRMS.spatial = t.ints[1]; m.tipRMS.act = t.ints[2];
    if(m.tipRMS.C != m.trunkC || t.nFloats != (uint32_t)(2 * m.trunkC + 1)) fail("trunk tip rmsnorm shape mismatch");
    m.tipRMS.eps = t.floats[0];
    m.tipRMS.gamma.assign(t.floats + 1, t.floats + 1 + m.trunkC);
    m.tipRMS.beta.assign(t.floats + 1 + m.trunkC, t.floats + 1 + 2 * m.trunkC);
  }
  else fail("unknown trunk norm kind");

  r = rd.expect(KB_TAG_POLICYHEAD, 3, "POLICYHEAD");
  if(r.ints[1] != m.policyC) fail("policy head channel count mismatch");
  m.hasPassMlp = r.ints[2];
  parseConv(rd, m.p1Conv); parseConv(rd, m.g1Conv); parseBN(rd, m.g1BN); parseMatMul(rd, m.gpoolToBias);
  parseBN(rd, m.p1BN); parseConv(rd, m.p2Conv); parseMatMul(rd, m.passMul);
  if(m.hasPassMlp) { parseMatBias(rd, m.passBias); m.passAct = parseAct(rd); parseMatMul(rd, m.passMul2); }
  if(m.p1Conv.inC != m.trunkC || m.g1Conv.inC != m.trunkC || m.p1Conv.outC != m.p1BN.C || m.g1Conv.outC != m.g1BN.C ||
     m.gpoolToBias.inC != 3 * m.g1BN.C || m.gpoolToBias.outC != m.p1BN.C || m.p2Conv.inC != m.p1BN.C ||
     m.p2Conv.outC != m.policyC || m.passMul.inC != 3 * m.g1BN.C)
    fail("policy head shape mismatch");
  if(m.p1Conv.kY != 1 || m.p1Conv.kX != 1 || m.g1Conv.kY != 1 || m.g1Conv.kX != 1 || m.p2Conv.kY != 1 || m.p2Conv.kX != 1)
    fail("policy head convolutions must be 1x1");
  if(m.hasPassMlp ? (m.passMul.outC != m.passBias.C || m.passMul2.inC != m.passMul.outC || m.passMul2.outC != m.policyC)
                  : (m.passMul.outC != m.policyC))
    fail("policy head pass shape mismatch");

  rd.expect(KB_TAG_VALUEHEAD, 1, "VALUEHEAD");
  parseConv(rd, m.v1Conv); parseBN(rd, m.v1BN); parseMatMul(rd, m.v2Mul); parseMatBias(rd, m.v2Bias); m.v2Act = parseAct(rd);
  parseMatMul(rd, m.v3Mul); parseMatBias(rd, m.v3Bias); parseMatMul(rd, m.sv3Mul); parseMatBias(rd, m.sv3Bias); parseConv(rd, m.ownConv);
  if(m.v1Conv.inC != m.trunkC || m.v1Conv.outC != m.v1BN.C || m.v2Mul.inC != 3 * m.v1BN.C || m.v2Mul.outC != m.v2Bias.C ||
     m.v3Mul.inC != m.v2Mul.outC || m.v3Mul.outC != m.v3Bias.C || m.v3Mul.outC != m.valueC || m.sv3Mul.inC != m.v2Mul.outC ||
     m.sv3Mul.outC != m.sv3Bias.C || m.sv3Mul.outC != m.scoreValueC || m.ownConv.inC != m.v1BN.C || m.ownConv.outC != m.ownershipC ||
     m.ownershipC != 1)
    fail("value head shape mismatch");
  if(m.v1Conv.kY != 1 || m.v1Conv.kX != 1 || m.ownConv.kY != 1 || m.ownConv.kX != 1) fail("value head convolutions must be 1x1");
  rd.expect(KB_TAG_END, 0, "END");
}

}  // namespace kb
