/* Model extension file: weights that the reference's model file format has no field for.
 *
 * The reference's format (cpp/neuralnet/desc.cpp:1094-1176 for an attention block) and its exporter
 * (python/export_model_pytorch.py) cannot carry a learned relative-position attention bias.  A net that has one is
 * therefore stored as an ordinary model file (every other weight; loadable by the reference's loader as it is) plus
 * an extension file next to it, named <model file>.kbext.  Backends that know the extension (the B200 backend and the
 * oracle's test backend) look for that file when they load a model and attach its records to the parsed ModelDesc by
 * block name while flattening it (modeldesc_blob.h); a model without the file loads exactly as before.
 *
 * Encoding (little-endian, every field a multiple of 4 bytes):
 *   header : 8 bytes "KBMDLEXT", u32 formatVersion (= 1), u32 nameBytes, model name (ModelDesc::name, zero-padded to a
 *            multiple of 4), u32 numRecords
 *   record : u32 kind, u32 payloadBytes, payload
 *   kind 1 (attention relative-position bias):
 *            u32 nameBytes, block name (TransformerAttentionDesc::name, zero-padded), u32 heads, u32 Y, u32 X,
 *            f32 table[heads][2Y-1][2X-1]   -- added to the scaled scores of query (yq,xq) and key (yk,xk) as
 *            table[head][yk-yq+Y-1][xk-xq+X-1] (the ATTNBIAS record of include/kb_modelblob.h)
 * A reader rejects a file whose version or model name differs, whose records run past the end, that names a block the
 * model does not have, or that holds a kind it does not know (a newer writer bumps formatVersion for new kinds).
 */
#ifndef KATAGO_B200_HOST_MODEL_EXT_H_
#define KATAGO_B200_HOST_MODEL_EXT_H_

#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <vector>

#include "core/global.h"

namespace kbhost {

struct AttnBiasExt {
  int heads = 0, Y = 0, X = 0;
  std::vector<float> table;
};

struct ModelExt {
  std::map<std::string, AttnBiasExt> attnBias;  // by attention block name
  bool empty() const { return attnBias.empty(); }
};

inline std::string modelExtPath(const std::string& modelFile) { return modelFile + ".kbext"; }

namespace ext_detail {
struct Cursor {
  const std::vector<char>& buf;
  size_t pos;
  const std::string& file;
  uint32_t u32() {
    if(pos + 4 > buf.size()) throw StringError(file + ": model extension file is truncated");
    uint32_t v;
    std::memcpy(&v, buf.data() + pos, 4);
    pos += 4;
    return v;
  }
  std::string str() {
    const uint32_t n = u32();
    const size_t padded = ((size_t)n + 3) / 4 * 4;
    if(n > 4096 || pos + padded > buf.size()) throw StringError(file + ": model extension file holds a malformed name");
    std::string s(buf.data() + pos, n);
    pos += padded;
    return s;
  }
};
}  // namespace ext_detail

// Reads <modelFile>.kbext if there is one.  Returns false (ext untouched) when the file does not exist; throws
// StringError when it exists and is malformed or belongs to another model.
inline bool loadModelExt(const std::string& modelFile, const std::string& modelName, ModelExt& ext) {
  const std::string file = modelExtPath(modelFile);
  std::ifstream in(file, std::ios::binary);
  if(!in.good()) return false;
  std::vector<char> buf((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  if(buf.size() < 20 || std::memcmp(buf.data(), "KBMDLEXT", 8) != 0) throw StringError(file + ": not a model extension file");
  ext_detail::Cursor c{buf, 8, file};
  const uint32_t version = c.u32();
  if(version != 1) throw StringError(file + ": model extension format version " + Global::uint32ToString(version) + " is not supported (this reader knows 1)");
  const std::string name = c.str();
  if(name != modelName) throw StringError(file + ": written for model '" + name + "', but the model file holds '" + modelName + "'");
  const uint32_t numRecords = c.u32();
  for(uint32_t r = 0; r < numRecords; r++) {
    const uint32_t kind = c.u32();
    const uint32_t payloadBytes = c.u32();
    if((payloadBytes % 4) != 0 || c.pos + payloadBytes > buf.size()) throw StringError(file + ": record runs past the end of the file");
    const size_t end = c.pos + payloadBytes;
    if(kind != 1) throw StringError(file + ": unknown record kind " + Global::uint32ToString(kind));
    const std::string block = c.str();
    AttnBiasExt b;
    b.heads = (int)c.u32(); b.Y = (int)c.u32(); b.X = (int)c.u32();
    if(b.heads < 1 || b.heads > 1024 || b.Y < 1 || b.Y > 64 || b.X < 1 || b.X > 64) throw StringError(file + ": attention bias of block '" + block + "' has an invalid shape");
    const size_t n = (size_t)b.heads * (2 * b.Y - 1) * (2 * b.X - 1);
    if(c.pos + n * 4 != end) throw StringError(file + ": attention bias of block '" + block + "' does not match its record length");
    b.table.resize(n);
    std::memcpy(b.table.data(), buf.data() + c.pos, n * 4);
    c.pos = end;
    if(!ext.attnBias.emplace(block, std::move(b)).second) throw StringError(file + ": two attention bias records for block '" + block + "'");
  }
  if(c.pos != buf.size()) throw StringError(file + ": bytes after the last record");
  return true;
}

}  // namespace kbhost

#endif
