/* ModelDesc -> model blob.  Host-side C++ that walks the reference's parsed model
 * (cpp/neuralnet/desc.h) and serialises it in the order and encoding documented in
 * include/kb_modelblob.h.  Compiled against the reference's headers (-I<reference>/cpp);
 * used by the B200 backend (b200backend.cpp) and by the oracle's test backend.
 */
#ifndef KATAGO_B200_HOST_MODELDESC_BLOB_H_
#define KATAGO_B200_HOST_MODELDESC_BLOB_H_

#include "neuralnet/desc.h"
#include "core/global.h"
#include "kb_modelblob.h"
#include "model_ext.h"

namespace kbhost {

// Extension records (model_ext.h) to attach while flattening, and how many of them found their block.
struct ExtAttach {
  const ModelExt* ext = nullptr;
  int attnBiasUsed = 0;
};

inline void writeConv(kbblob::Writer& w, const ConvLayerDesc& d) {
  w.record(KB_TAG_CONV, {d.convYSize, d.convXSize, d.inChannels, d.outChannels, d.dilationY, d.dilationX}, d.weights);
}

// A batch norm and the activation that follows it travel as one record holding the
// merged per-channel scale and bias (desc.cpp:278-285).
inline void writeBN(kbblob::Writer& w, const BatchNormLayerDesc& d, int activation) {
  std::vector<float> f;
  f.reserve(2 * (size_t)d.numChannels);
  f.insert(f.end(), d.mergedScale.begin(), d.mergedScale.end());
  f.insert(f.end(), d.mergedBias.begin(), d.mergedBias.end());
  w.record(KB_TAG_BN, {d.numChannels, activation}, f);
}

inline void writeMatMul(kbblob::Writer& w, const MatMulLayerDesc& d) {
  w.record(KB_TAG_MATMUL, {d.inChannels, d.outChannels}, d.weights);
}

inline void writeMatBias(kbblob::Writer& w, const MatBiasLayerDesc& d) {
  w.record(KB_TAG_MATBIAS, {d.numChannels}, d.weights);
}

inline void writeAct(kbblob::Writer& w, const ActivationLayerDesc& d) {
  w.record(KB_TAG_ACT, {d.activation});
}

inline void writeTRMSNorm(kbblob::Writer& w, const TransformerRMSNormDesc& d) {
  std::vector<float> f;
  f.push_back(d.epsilon);
  f.insert(f.end(), d.weight.begin(), d.weight.end());
  w.record(KB_TAG_TRMSNORM, {d.numChannels}, f);
}

inline void writeBlocks(kbblob::Writer& w, const std::vector<std::pair<int, unique_ptr_void>>& blocks, ExtAttach* ea = nullptr);

inline void writeOrdinaryBlock(kbblob::Writer& w, const ResidualBlockDesc& d) {
  w.record(KB_TAG_BLOCK_ORDINARY, {});
  writeBN(w, d.preBN, d.preActivation.activation);
  writeConv(w, d.regularConv);
  writeBN(w, d.midBN, d.midActivation.activation);
  writeConv(w, d.finalConv);
}

inline void writeGPoolBlock(kbblob::Writer& w, const GlobalPoolingResidualBlockDesc& d) {
  w.record(KB_TAG_BLOCK_GPOOL, {});
  writeBN(w, d.preBN, d.preActivation.activation);
  writeConv(w, d.regularConv);
  writeConv(w, d.gpoolConv);
  writeBN(w, d.gpoolBN, d.gpoolActivation.activation);
  writeMatMul(w, d.gpoolToBiasMul);
  writeBN(w, d.midBN, d.midActivation.activation);
  writeConv(w, d.finalConv);
}

inline void writeNestedBlock(kbblob::Writer& w, const NestedBottleneckResidualBlockDesc& d, ExtAttach* ea = nullptr) {
  w.record(KB_TAG_BLOCK_NESTED, {d.numBlocks});
  writeBN(w, d.preBN, d.preActivation.activation);
  writeConv(w, d.preConv);
  writeBlocks(w, d.blocks, ea);
  writeBN(w, d.postBN, d.postActivation.activation);
  writeConv(w, d.postConv);
}

inline void writeAttnBlock(kbblob::Writer& w, const TransformerAttentionDesc& d, ExtAttach* ea = nullptr) {
  std::vector<float> f;
  if(d.useRope && d.learnableRope) f = d.ropeFreqs;
  else if(d.useRope) f.push_back(d.ropeTheta);
  w.record(
    KB_TAG_BLOCK_ATTN,
    {d.numHeads, d.numKVHeads, d.qHeadDim, d.vHeadDim, d.useRope ? 1 : 0, d.learnableRope ? 1 : 0}, f);
  writeTRMSNorm(w, d.preLN);
  writeMatMul(w, d.qProj);
  writeMatMul(w, d.kProj);
  writeMatMul(w, d.vProj);
  writeMatMul(w, d.outProj);
  if(ea && ea->ext) {
    auto it = ea->ext->attnBias.find(d.name);
    if(it != ea->ext->attnBias.end()) {
      const AttnBiasExt& b = it->second;
      if(b.heads != d.numHeads)
        throw StringError("model extension: attention bias of block '" + d.name + "' has " + Global::intToString(b.heads) + " heads, the block " + Global::intToString(d.numHeads));
      w.record(KB_TAG_ATTNBIAS, {b.heads, b.Y, b.X}, b.table);
      ea->attnBiasUsed++;
    }
  }
}

inline void writeFFNBlock(kbblob::Writer& w, const TransformerFFNDesc& d) {
  w.record(KB_TAG_BLOCK_FFN, {d.numChannels, d.ffnChannels, d.useSwiGLU ? 1 : 0});
  writeTRMSNorm(w, d.preLN);
  writeMatMul(w, d.linear1);
  if(d.useSwiGLU) writeMatMul(w, d.linearGate);
  writeMatMul(w, d.linear2);
}

inline void writeBlocks(kbblob::Writer& w, const std::vector<std::pair<int, unique_ptr_void>>& blocks, ExtAttach* ea) {
  for(const auto& b : blocks) {
    switch(b.first) {
      case ORDINARY_BLOCK_KIND: writeOrdinaryBlock(w, *(const ResidualBlockDesc*)b.second.get()); break;
      case GLOBAL_POOLING_BLOCK_KIND: writeGPoolBlock(w, *(const GlobalPoolingResidualBlockDesc*)b.second.get()); break;
      case NESTED_BOTTLENECK_BLOCK_KIND: writeNestedBlock(w, *(const NestedBottleneckResidualBlockDesc*)b.second.get(), ea); break;
      case TRANSFORMER_ATTENTION_BLOCK_KIND: writeAttnBlock(w, *(const TransformerAttentionDesc*)b.second.get(), ea); break;
      case TRANSFORMER_FFN_BLOCK_KIND: writeFFNBlock(w, *(const TransformerFFNDesc*)b.second.get()); break;
      default: throw StringError("b200 backend: unknown block kind " + Global::intToString(b.first));
    }
  }
}

// ext (or NULL): records of the model's extension file, attached to the blocks they name; every record must find its block.
inline std::vector<uint32_t> modelDescToBlob(const ModelDesc& m, const ModelExt* ext = nullptr) {
  kbblob::Writer w;
  ExtAttach ea;
  ea.ext = ext;
  w.record(
    KB_TAG_MODEL,
    {m.modelVersion, m.numInputChannels, m.numInputGlobalChannels, m.numInputMetaChannels, m.numPolicyChannels,
     m.numValueChannels, m.numScoreValueChannels, m.numOwnershipChannels});
  const TrunkDesc& t = m.trunk;
  w.record(
    KB_TAG_TRUNK,
    {t.numBlocks, t.trunkNumChannels, t.midNumChannels, t.regularNumChannels, t.gpoolNumChannels, t.trunkNormKind});
  writeConv(w, t.initialConv);
  writeMatMul(w, t.initialMatMul);
  if(m.numInputMetaChannels > 0) {
    // SGF metadata encoder of human-SL nets (desc.h SGFMetadataEncoderDesc)
    const SGFMetadataEncoderDesc& e = t.sgfMetadataEncoder;
    w.record(KB_TAG_METAENC, {e.metaEncoderVersion, e.numInputMetaChannels});
    writeMatMul(w, e.mul1); writeMatBias(w, e.bias1); writeAct(w, e.act1);
    writeMatMul(w, e.mul2); writeMatBias(w, e.bias2); writeAct(w, e.act2);
    writeMatMul(w, e.mul3);
  }
  writeBlocks(w, t.blocks, &ea);
  if(ext && ea.attnBiasUsed != (int)ext->attnBias.size())
    throw StringError("model extension: " + Global::intToString((int)ext->attnBias.size() - ea.attnBiasUsed) + " attention bias record(s) name a block that model '" + m.name + "' does not have");
  if(t.trunkNormKind == TRUNK_NORM_KIND_STANDARD) {
    writeBN(w, t.trunkTipBN, t.trunkTipActivation.activation);
  }
  else {
    const RMSNormLayerDesc& r = t.trunkTipRMSNorm;
    std::vector<float> f;
    f.push_back(r.epsilon);
    f.insert(f.end(), r.gamma.begin(), r.gamma.end());
    f.insert(f.end(), r.beta.begin(), r.beta.end());
    w.record(KB_TAG_RMSNORM, {r.numChannels, r.spatial ? 1 : 0, t.trunkTipActivation.activation}, f);
  }
  const PolicyHeadDesc& p = m.policyHead;
  const int hasPassMlp = m.modelVersion >= 15 ? 1 : 0;
  w.record(KB_TAG_POLICYHEAD, {m.modelVersion, p.policyOutChannels, hasPassMlp});
  writeConv(w, p.p1Conv);
  writeConv(w, p.g1Conv);
  writeBN(w, p.g1BN, p.g1Activation.activation);
  writeMatMul(w, p.gpoolToBiasMul);
  writeBN(w, p.p1BN, p.p1Activation.activation);
  writeConv(w, p.p2Conv);
  writeMatMul(w, p.gpoolToPassMul);
  if(hasPassMlp) {
    writeMatBias(w, p.gpoolToPassBias);
    writeAct(w, p.passActivation);
    writeMatMul(w, p.gpoolToPassMul2);
  }
  const ValueHeadDesc& v = m.valueHead;
  w.record(KB_TAG_VALUEHEAD, {m.modelVersion});
  writeConv(w, v.v1Conv);
  writeBN(w, v.v1BN, v.v1Activation.activation);
  writeMatMul(w, v.v2Mul);
  writeMatBias(w, v.v2Bias);
  writeAct(w, v.v2Activation);
  writeMatMul(w, v.v3Mul);
  writeMatBias(w, v.v3Bias);
  writeMatMul(w, v.sv3Mul);
  writeMatBias(w, v.sv3Bias);
  writeConv(w, v.vOwnershipConv);
  w.record(KB_TAG_END, {});
  return w.finish();
}

// Single-layer blobs for the reference's layer tests (nninterface.h:134-180).
inline std::vector<uint32_t> convToBlob(const ConvLayerDesc& d) {
  kbblob::Writer w; writeConv(w, d); return w.finish();
}
inline std::vector<uint32_t> bnToBlob(const BatchNormLayerDesc& d, int activation) {
  kbblob::Writer w; writeBN(w, d, activation); return w.finish();
}
inline std::vector<uint32_t> ordinaryBlockToBlob(const ResidualBlockDesc& d) {
  kbblob::Writer w; writeOrdinaryBlock(w, d); return w.finish();
}
inline std::vector<uint32_t> gpoolBlockToBlob(const GlobalPoolingResidualBlockDesc& d) {
  kbblob::Writer w; writeGPoolBlock(w, d); return w.finish();
}

// NCHW <-> NHWC helpers for the layer tests, which may hand either layout.
inline std::vector<float> nchwToNhwc(const std::vector<float>& in, int n, int c, int h, int w) {
  std::vector<float> out(in.size());
  for(int b = 0; b < n; b++)
    for(int ch = 0; ch < c; ch++)
      for(int y = 0; y < h; y++)
        for(int x = 0; x < w; x++)
          out[(((size_t)b * h + y) * w + x) * c + ch] = in[(((size_t)b * c + ch) * h + y) * w + x];
  return out;
}
inline std::vector<float> nhwcToNchw(const std::vector<float>& in, int n, int c, int h, int w) {
  std::vector<float> out(in.size());
  for(int b = 0; b < n; b++)
    for(int ch = 0; ch < c; ch++)
      for(int y = 0; y < h; y++)
        for(int x = 0; x < w; x++)
          out[(((size_t)b * c + ch) * h + y) * w + x] = in[(((size_t)b * h + y) * w + x) * c + ch];
  return out;
}

}  // namespace kbhost

#endif
