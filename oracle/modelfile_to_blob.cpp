/* Test helper: loads a KataGo model file with the reference's own loader
 * (ModelDesc::loadFromFileMaybeGZipped, cpp/neuralnet/desc.cpp:2574-2636) and writes the
 * model blob produced by katago_b200/host/modeldesc_blob.h.  Used to check the Python
 * model-file reader and blob writer against the reference's parser.  TEST INFRASTRUCTURE ONLY.
 *
 * usage: modelfile_to_blob MODEL_FILE OUT_BLOB
 */
#include "neuralnet/desc.h"
#include "core/global.h"
#include "modeldesc_blob.h"

#include <cstdio>
#include <iostream>

int main(int argc, char** argv) {
  if(argc != 3) {
    std::cerr << "usage: modelfile_to_blob MODEL_FILE OUT_BLOB" << std::endl;
    return 2;
  }
  try {
    ModelDesc desc;
    ModelDesc::loadFromFileMaybeGZipped(argv[1], desc, "");
    kbhost::ModelExt ext;  // MODEL_FILE.kbext, if there is one, as the backends attach it
    kbhost::loadModelExt(argv[1], desc.name, ext);
    std::vector<uint32_t> blob = kbhost::modelDescToBlob(desc, ext.empty() ? nullptr : &ext);
    FILE* f = std::fopen(argv[2], "wb");
    if(f == NULL) { std::cerr << "cannot open output" << std::endl; return 1; }
    std::fwrite(blob.data(), 4, blob.size(), f);
    std::fclose(f);
    std::cout << desc.name << " version " << desc.modelVersion << " words " << blob.size() << std::endl;
  }
  catch(const StringError& e) {
    std::cerr << e.what() << std::endl;
    return 1;
  }
  return 0;
}
