/* nninterface.h backend over the CPU oracle.  TEST INFRASTRUCTURE ONLY.
 *
 * Purpose: let the reference's own, unmodified test programs (runnnlayertests,
 * runtinynntests, testgpuerror, ...) run against oracle/kata_oracle.cpp, which pins
 * the oracle to the reference's known-answer vectors, and lets `testgpuerror
 * -reference-file` write the fp32 reference values that other backends are compared
 * with.  Built by oracle/Makefile against the reference sources where they lie; it is
 * compiled with -DUSE_EIGEN_BACKEND so that the reference's callers treat it exactly
 * like their CPU backend (fp32 only, NHWC only).
 */
#include "neuralnet/nninterface.h"
#include "neuralnet/nneval.h"
#include "neuralnet/modelversion.h"

#include "kata_oracle.h"
#include "modeldesc_blob.h"
#include "nnoutput_glue.h"

using namespace std;

struct LoadedModel {
  ModelDesc modelDesc;
  kbhost::ModelExt ext;  // records of <model file>.kbext, if there is one (katago_b200/host/model_ext.h)
  LoadedModel(const string& fileName, const string& expectedSha256) {
    ModelDesc::loadFromFileMaybeGZipped(fileName, modelDesc, expectedSha256);
    kbhost::loadModelExt(fileName, modelDesc.name, ext);
  }
};

struct ComputeContext {
  int nnXLen;
  int nnYLen;
};

struct ComputeHandle {
  ko_model* model = nullptr;
  kbhost::NetDims dims;
  bool inputsUseNHWC = true;
  ~ComputeHandle() { ko_model_destroy(model); }
};

struct InputBuffers {
  int maxBatchSize;
  size_t singleInputElts;
  size_t metaChannels = 0;
  vector<float> spatial, global, meta, scratch;
  vector<float> policy, policyPass, value, scoreValue, ownership;
};

static void check(int status, const char* what) {
  if(status != 0)
    throw StringError(string("oracle backend: ") + what + ": " + ko_last_error());
}

void NeuralNet::globalInitialize() {}
void NeuralNet::globalCleanup() {}
void NeuralNet::printDevices() {}

LoadedModel* NeuralNet::loadModelFile(const string& file, const string& expectedSha256) {
  return new LoadedModel(file, expectedSha256);
}
void NeuralNet::freeLoadedModel(LoadedModel* loadedModel) { delete loadedModel; }
const ModelDesc& NeuralNet::getModelDesc(const LoadedModel* loadedModel) { return loadedModel->modelDesc; }

ComputeContext* NeuralNet::createComputeContext(
  const std::vector<int>& gpuIdxs, Logger* logger, int nnXLen, int nnYLen, const string& homeDataDirOverride,
  enabled_t useFP16Mode, const LoadedModel* loadedModel, ConfigParser& cfg) {
  (void)gpuIdxs; (void)logger; (void)homeDataDirOverride; (void)loadedModel; (void)cfg;
  if(useFP16Mode == enabled_t::True)
    throw StringError("oracle backend: useFP16 = true not supported");
  return new ComputeContext{nnXLen, nnYLen};
}
void NeuralNet::freeComputeContext(ComputeContext* computeContext) { delete computeContext; }

ComputeHandle* NeuralNet::createComputeHandle(
  ComputeContext* context, const LoadedModel* loadedModel, Logger* logger, int maxBatchSize, bool requireExactNNLen,
  bool inputsUseNHWC, int gpuIdxForThisThread, int serverThreadIdx) {
  (void)maxBatchSize; (void)requireExactNNLen; (void)gpuIdxForThisThread;
  if(logger != NULL)
    logger->write("Oracle (CPU) backend thread " + Global::intToString(serverThreadIdx) + ": Model name: " + loadedModel->modelDesc.name);
  auto handle = std::make_unique<ComputeHandle>();
  handle->dims = kbhost::makeNetDims(loadedModel->modelDesc, context->nnXLen, context->nnYLen);
  handle->inputsUseNHWC = inputsUseNHWC;
  std::vector<uint32_t> blob = kbhost::modelDescToBlob(loadedModel->modelDesc, loadedModel->ext.empty() ? nullptr : &loadedModel->ext);
  check(ko_model_create(blob.data(), blob.size() * 4, context->nnXLen, context->nnYLen, &handle->model), "ko_model_create");
  return handle.release();
}
void NeuralNet::freeComputeHandle(ComputeHandle* gpuHandle) { delete gpuHandle; }
bool NeuralNet::isUsingFP16(const ComputeHandle* handle) { (void)handle; return false; }
bool NeuralNet::setIsWarmup(const ComputeHandle* handle, bool isWarmup) { (void)handle; (void)isWarmup; return false; }

InputBuffers* NeuralNet::createInputBuffers(const LoadedModel* loadedModel, int maxBatchSize, int nnXLen, int nnYLen) {
  const ModelDesc& m = loadedModel->modelDesc;
  const size_t S = (size_t)nnXLen * nnYLen;
  InputBuffers* b = new InputBuffers();
  b->maxBatchSize = maxBatchSize;
  b->singleInputElts = S * m.numInputChannels;
  b->spatial.resize(b->singleInputElts * maxBatchSize);
  b->scratch.resize(b->singleInputElts);
  b->global.resize((size_t)m.numInputGlobalChannels * maxBatchSize);
  b->metaChannels = (size_t)m.numInputMetaChannels;
  b->meta.resize(b->metaChannels * maxBatchSize);
  b->policy.resize(S * m.numPolicyChannels * maxBatchSize);
  b->policyPass.resize((size_t)m.numPolicyChannels * maxBatchSize);
  b->value.resize((size_t)m.numValueChannels * maxBatchSize);
  b->scoreValue.resize((size_t)m.numScoreValueChannels * maxBatchSize);
  b->ownership.resize(S * maxBatchSize);
  return b;
}
void NeuralNet::freeInputBuffers(InputBuffers* buffers) { delete buffers; }

// NNResultBuf -> one row of the contiguous NHWC spatial / global staging arrays, applying the row's board symmetry on the
// host (nninputs.cpp:529-597).  inputsUseNHWC describes the layout of rowSpatialBuf; the staging row is always NHWC.
static void packRow(
  const kbhost::NetDims& d, const NNResultBuf* buf, bool inputsUseNHWC, float* spatialRowNHWC, float* globalRow, float* scratchRow) {
  const int S = d.nnXLen * d.nnYLen;
  const int C = d.numSpatialFeatures;
  std::copy(buf->rowGlobalBuf.begin(), buf->rowGlobalBuf.begin() + d.numGlobalFeatures, globalRow);
  if(inputsUseNHWC) {
    SymmetryHelpers::copyInputsWithSymmetry(buf->rowSpatialBuf.data(), spatialRowNHWC, 1, d.nnYLen, d.nnXLen, C, true, buf->symmetry);
  }
  else {
    SymmetryHelpers::copyInputsWithSymmetry(buf->rowSpatialBuf.data(), scratchRow, 1, d.nnYLen, d.nnXLen, C, false, buf->symmetry);
    for(int c = 0; c < C; c++)
      for(int s = 0; s < S; s++)
        spatialRowNHWC[(size_t)s * C + c] = scratchRow[(size_t)c * S + s];
  }
}

void NeuralNet::getOutput(
  ComputeHandle* h, InputBuffers* b, int numBatchEltsFilled, NNResultBuf** inputBufs, vector<NNOutput*>& outputs) {
  const int n = numBatchEltsFilled;
  if(n <= 0 || n > b->maxBatchSize || (int)outputs.size() != n)
    throw StringError("oracle backend: bad batch size in getOutput");
  const kbhost::NetDims& d = h->dims;
  const size_t S = (size_t)d.nnXLen * d.nnYLen;
  for(int row = 0; row < n; row++)
    packRow(
      d, inputBufs[row], h->inputsUseNHWC, b->spatial.data() + b->singleInputElts * row,
      b->global.data() + (size_t)d.numGlobalFeatures * row, b->scratch.data());
  // SGF metadata rows exactly for nets with the encoder (eigenbackend.cpp:2462-2472)
  for(int row = 0; row < n; row++) {
    if((b->metaChannels > 0) != inputBufs[row]->hasRowMeta)
      throw StringError("oracle backend: SGF metadata rows must be given exactly for models with a metadata encoder");
    if(b->metaChannels > 0)
      std::copy(inputBufs[row]->rowMetaBuf.begin(), inputBufs[row]->rowMetaBuf.begin() + b->metaChannels, b->meta.begin() + b->metaChannels * row);
  }
  check(
    ko_forward_meta(
      h->model, n, b->spatial.data(), b->global.data(), b->metaChannels > 0 ? b->meta.data() : nullptr, b->policy.data(),
      b->policyPass.data(), b->value.data(), b->scoreValue.data(), b->ownership.data(), nullptr),
    "ko_forward_meta");
  for(int row = 0; row < n; row++)
    kbhost::unpackRow(
      d, inputBufs[row], outputs[row], b->policy.data() + S * d.numPolicyChannels * row,
      b->policyPass.data() + (size_t)d.numPolicyChannels * row, b->value.data() + (size_t)d.numValueChannels * row,
      b->scoreValue.data() + (size_t)d.numScoreValueChannels * row, b->ownership.data() + S * row);
}

// Layer tests ---------------------------------------------------------------------------------------

static bool evalLayer(
  const std::vector<uint32_t>& blob, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC, int inC, int outC,
  const std::vector<float>& inputBuffer, const std::vector<float>* maskBuffer, std::vector<float>& outputBuffer) {
  if(useFP16)
    return false;
  std::vector<float> in = useNHWC ? inputBuffer : kbhost::nchwToNhwc(inputBuffer, batchSize, inC, nnYLen, nnXLen);
  std::vector<float> out((size_t)batchSize * nnXLen * nnYLen * outC);
  check(
    ko_eval_layer(blob.data(), blob.size() * 4, batchSize, nnXLen, nnYLen, in.data(), maskBuffer ? maskBuffer->data() : nullptr, out.data()),
    "ko_eval_layer");
  outputBuffer = useNHWC ? out : kbhost::nhwcToNchw(out, batchSize, outC, nnYLen, nnXLen);
  return true;
}

bool NeuralNet::testEvaluateConv(
  const ConvLayerDesc* desc, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC,
  const std::vector<float>& inputBuffer, std::vector<float>& outputBuffer) {
  return evalLayer(kbhost::convToBlob(*desc), batchSize, nnXLen, nnYLen, useFP16, useNHWC, desc->inChannels, desc->outChannels, inputBuffer, nullptr, outputBuffer);
}

bool NeuralNet::testEvaluateBatchNorm(
  const BatchNormLayerDesc* desc, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC,
  const std::vector<float>& inputBuffer, const std::vector<float>& maskBuffer, std::vector<float>& outputBuffer) {
  return evalLayer(kbhost::bnToBlob(*desc, ACTIVATION_IDENTITY), batchSize, nnXLen, nnYLen, useFP16, useNHWC, desc->numChannels, desc->numChannels, inputBuffer, &maskBuffer, outputBuffer);
}

bool NeuralNet::testEvaluateResidualBlock(
  const ResidualBlockDesc* desc, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC,
  const std::vector<float>& inputBuffer, const std::vector<float>& maskBuffer, std::vector<float>& outputBuffer) {
  int c = desc->preBN.numChannels;
  return evalLayer(kbhost::ordinaryBlockToBlob(*desc), batchSize, nnXLen, nnYLen, useFP16, useNHWC, c, c, inputBuffer, &maskBuffer, outputBuffer);
}

bool NeuralNet::testEvaluateGlobalPoolingResidualBlock(
  const GlobalPoolingResidualBlockDesc* desc, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC,
  const std::vector<float>& inputBuffer, const std::vector<float>& maskBuffer, std::vector<float>& outputBuffer) {
  int c = desc->preBN.numChannels;
  return evalLayer(kbhost::gpoolBlockToBlob(*desc), batchSize, nnXLen, nnYLen, useFP16, useNHWC, c, c, inputBuffer, &maskBuffer, outputBuffer);
}
