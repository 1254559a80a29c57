/* Flat binary description of a KataGo network ("model blob").
 *
 * The blob is what crosses the C ABI when a model is handed to the B200 library
 * (kb_model_create) or to the CPU oracle (ko_model_create).  It is the content of
 * the reference's ModelDesc tree (cpp/neuralnet/desc.h:15-537) AFTER parsing and
 * after batch-norm merging (desc.cpp:278-285), flattened in the order in which
 * the reference's model file lists the layers (desc.cpp:2280-2443).  The host
 * side (C++ over ModelDesc, or Python over the model file) writes it; the
 * libraries read it.
 *
 * Encoding: little-endian 32-bit words.
 *   header : u32 magic 'KBM1', u32 formatVersion (=1), u32 totalWords
 *   record : u32 tag, u32 nInts, i32 ints[nInts], u32 nFloats, f32 floats[nFloats]
 *
 * Grammar (each name is one record with the given ints / floats):
 *   model       := MODEL{modelVersion,inC,inGlobalC,inMetaC,policyC,valueC,scoreValueC,ownershipC}
 *                  trunk policyhead valuehead END
 *   trunk       := TRUNK{numBlocks,trunkC,midC,regularC,gpoolC,normKind}
 *                  CONV MATMUL [inMetaC > 0: METAENC{metaEncoderVersion,inMetaC} MATMUL MATBIAS ACT MATMUL MATBIAS ACT MATMUL]
 *                  block*numBlocks (BN | RMSNORM)
 *                  (METAENC: the SGF metadata encoder of human-SL nets, desc.cpp:1476-1522; its output [n][trunkC] is
 *                  added to the trunk like the global-feature bias, eigenbackend.cpp:1917-1920)
 *   block       := BLOCK_ORDINARY BN CONV BN CONV
 *                | BLOCK_GPOOL BN CONV(regular) CONV(gpool) BN(gpool) MATMUL BN(mid) CONV(final)
 *                | BLOCK_NESTED{numInner} BN CONV block*numInner BN CONV
 *                | BLOCK_ATTN{heads,kvHeads,qDim,vDim,useRope,learnableRope,ropePairs}[theta, freqs...]
 *                  TRMSNORM MATMUL(q) MATMUL(k) MATMUL(v) MATMUL(out) [ATTNBIAS{heads,Y,X}[heads*(2Y-1)*(2X-1)]]
 *                  (ATTNBIAS: optional learned relative-position bias, added to the scaled scores of query (yq,xq)
 *                  and key (yk,xk) as table[head][yk-yq+Y-1][xk-xq+X-1]; an extension of this library, the
 *                  reference's model files cannot carry it)
 *                | BLOCK_FFN{C,ffnC,useSwiGLU} TRMSNORM MATMUL(1) [MATMUL(gate)] MATMUL(2)
 *   policyhead  := POLICYHEAD{modelVersion,policyC,hasPassMlp} CONV(p1) CONV(g1) BN(g1) MATMUL(gpoolToBias)
 *                  BN(p1) CONV(p2) MATMUL(pass) [hasPassMlp: MATBIAS ACT MATMUL(pass2)]
 *   valuehead   := VALUEHEAD{modelVersion} CONV(v1) BN(v1) MATMUL(v2) MATBIAS ACT MATMUL(v3) MATBIAS
 *                  MATMUL(sv3) MATBIAS CONV(ownership)
 *   CONV        := {kY,kX,inC,outC,dilY,dilX} weights[oc][ic][y][x]      (desc.h:23)
 *   BN          := {C,activation} mergedScale[C] mergedBias[C]           (BN + the activation that follows it)
 *   MATMUL      := {inC,outC} weights[ic][oc]                            (desc.h:95)
 *   MATBIAS     := {C} bias[C]
 *   ACT         := {activation}
 *   RMSNORM     := {C,spatial,activation} [eps, gamma[C], beta[C]]
 *   TRMSNORM    := {C} [eps, weight[C]]
 * Activation codes are the reference's (neuralnet/activations.h).
 */
#ifndef KB_MODELBLOB_H_
#define KB_MODELBLOB_H_

#include <stdint.h>

#define KB_BLOB_MAGIC 0x314D424Bu /* "KBM1" */
#define KB_BLOB_FORMAT_VERSION 1u

enum {
  KB_TAG_MODEL = 1,
  KB_TAG_TRUNK = 2,
  KB_TAG_CONV = 3,
  KB_TAG_BN = 4,
  KB_TAG_MATMUL = 5,
  KB_TAG_MATBIAS = 6,
  KB_TAG_ACT = 7,
  KB_TAG_BLOCK_ORDINARY = 10,
  KB_TAG_BLOCK_GPOOL = 11,
  KB_TAG_BLOCK_NESTED = 12,
  KB_TAG_BLOCK_ATTN = 13,
  KB_TAG_BLOCK_FFN = 14,
  KB_TAG_RMSNORM = 15,
  KB_TAG_TRMSNORM = 16,
  KB_TAG_ATTNBIAS = 17,
  KB_TAG_POLICYHEAD = 20,
  KB_TAG_VALUEHEAD = 21,
  KB_TAG_METAENC = 22,
  KB_TAG_END = 99
};

enum {
  KB_ACT_IDENTITY = 0,
  KB_ACT_RELU = 1,
  KB_ACT_MISH = 2,
  KB_ACT_SILU = 3,
  KB_ACT_MISH_SCALE8 = 12
};

#ifdef __cplusplus
#include <cstring>
#include <string>
#include <vector>
#include <stdexcept>

namespace kbblob {

/* One decoded record; pointers alias the blob. */
struct Record {
  uint32_t tag = 0;
  uint32_t nInts = 0;
  const int32_t* ints = nullptr;
  uint32_t nFloats = 0;
  const float* floats = nullptr;
};

/* Sequential reader with bounds checks; throws std::runtime_error on malformed input. */
class Reader {
 public:
  Reader(const void* blob, size_t nbytes) {
    if(blob == nullptr || nbytes < 12 || (nbytes % 4) != 0)
      throw std::runtime_error("model blob: too small or not a multiple of 4 bytes");
    words_ = static_cast<const uint32_t*>(blob);
    nWords_ = nbytes / 4;
    if(words_[0] != KB_BLOB_MAGIC)
      throw std::runtime_error("model blob: bad magic");
    if(words_[1] != KB_BLOB_FORMAT_VERSION)
      throw std::runtime_error("model blob: unsupported format version");
    if(words_[2] != nWords_)
      throw std::runtime_error("model blob: length field does not match buffer size");
    pos_ = 3;
  }
  uint32_t peekTag() const {
    if(pos_ >= nWords_) throw std::runtime_error("model blob: truncated (peek)");
    return words_[pos_];
  }
  Record next() {
    Record r;
    need(2);
    r.tag = words_[pos_++];
    r.nInts = words_[pos_++];
    need(r.nInts);
    r.ints = reinterpret_cast<const int32_t*>(words_ + pos_);
    pos_ += r.nInts;
    need(1);
    r.nFloats = words_[pos_++];
    need(r.nFloats);
    r.floats = reinterpret_cast<const float*>(words_ + pos_);
    pos_ += r.nFloats;
    return r;
  }
  Record expect(uint32_t tag, uint32_t minInts, const char* what) {
    Record r = next();
    if(r.tag != tag)
      throw std::runtime_error(std::string("model blob: expected ") + what + " record, found tag " + std::to_string(r.tag));
    if(r.nInts < minInts)
      throw std::runtime_error(std::string("model blob: ") + what + " record has too few ints");
    return r;
  }
  bool atEnd() const { return pos_ >= nWords_; }

 private:
  void need(size_t n) const {
    if(pos_ + n > nWords_) throw std::runtime_error("model blob: truncated");
  }
  const uint32_t* words_;
  size_t nWords_;
  size_t pos_;
};

/* Writer used by the C++ host side. */
class Writer {
 public:
  Writer() { words_.assign(3, 0u); }
  void record(uint32_t tag, const std::vector<int32_t>& ints, const float* floats, size_t nFloats) {
    words_.push_back(tag);
    words_.push_back((uint32_t)ints.size());
    for(int32_t v : ints) words_.push_back((uint32_t)v);
    words_.push_back((uint32_t)nFloats);
    size_t at = words_.size();
    words_.resize(at + nFloats);
    if(nFloats > 0) std::memcpy(words_.data() + at, floats, nFloats * sizeof(float));
  }
  void record(uint32_t tag, const std::vector<int32_t>& ints) { record(tag, ints, nullptr, 0); }
  void record(uint32_t tag, const std::vector<int32_t>& ints, const std::vector<float>& floats) {
    record(tag, ints, floats.data(), floats.size());
  }
  const std::vector<uint32_t>& finish() {
    words_[0] = KB_BLOB_MAGIC;
    words_[1] = KB_BLOB_FORMAT_VERSION;
    words_[2] = (uint32_t)words_.size();
    return words_;
  }

 private:
  std::vector<uint32_t> words_;
};

}  // namespace kbblob
#endif /* __cplusplus */

#endif /* KB_MODELBLOB_H_ */
