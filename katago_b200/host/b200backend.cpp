/* KataGo neural-net backend for NVIDIA B200 (sm_100a).
 *
 * Implements the reference's backend contract, cpp/neuralnet/nninterface.h:32-182, on top of
 * the C ABI of libkatab200.so (include/katab200.h).  It takes the place of one of the
 * reference's backend translation units (cudabackend.cpp, eigenbackend.cpp, ...): compile it
 * with the rest of the reference's sources and link libkatab200.so.  NNEvaluator, search, GTP,
 * benchmark and testgpuerror run on it unchanged.
 *
 * Division of labour:
 *   - model file parsing stays with the reference's loader (ModelDesc, desc.cpp);
 *   - this file flattens the ModelDesc into a model blob (modeldesc_blob.h), stages rows in
 *     page-locked memory and unpacks results into NNOutput (nnoutput_glue.h);
 *   - everything numeric happens in the CUDA library; there is no CPU path.
 *
 * Precision: useFP16Mode True/Auto selects reduced precision (fp16 by default; the config key
 * `cudaPrecision = bf16` or the environment variable KATAB200_PRECISION=bf16 selects bfloat16),
 * False selects fp32.  isUsingFP16() reports true for both reduced modes so that testgpuerror
 * builds its fp32 twin evaluator (command/gputest.cpp:122-133).
 *
 * Built under -DUSE_CUDA_BACKEND so that the reference's callers use their CUDA-backend
 * branches (config key prefix "cuda", no transformer warm-up loop; program/setup.cpp:82-94,
 * neuralnet/nneval.cpp:481) with no edits to the reference.
 */
#include "neuralnet/nninterface.h"
#include "neuralnet/nneval.h"
#include "neuralnet/modelversion.h"

#include "katab200.h"
#include "modeldesc_blob.h"
#include "nnoutput_glue.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>

using namespace std;

static void check(int status, const char* what) {
  if(status != 0)
    throw StringError(string("B200 backend: ") + what + ": " + kb_last_error());
}

// LoadedModel -------------------------------------------------------------------------------------

struct LoadedModel {
  ModelDesc modelDesc;
  kbhost::ModelExt ext;  // records of <model file>.kbext, if there is one (model_ext.h)
  LoadedModel(const string& fileName, const string& expectedSha256) {
    ModelDesc::loadFromFileMaybeGZipped(fileName, modelDesc, expectedSha256);
    kbhost::loadModelExt(fileName, modelDesc.name, ext);
    // Same fp16 range trick as the reference's CUDA backend (cudabackend.cpp:3079-3082): activations of
    // Mish nets are carried at 1/8 scale, compensated by MISH_SCALE8 and postProcessParams.outputScaleMultiplier.
    // Done here because NNEvaluator copies postProcessParams right after loading (nneval.cpp:142).
    modelDesc.applyScale8ToReduceActivations();
  }
  LoadedModel() = delete;
  LoadedModel(const LoadedModel&) = delete;
  LoadedModel& operator=(const LoadedModel&) = delete;
};

LoadedModel* NeuralNet::loadModelFile(const string& file, const string& expectedSha256) {
  return new LoadedModel(file, expectedSha256);
}
void NeuralNet::freeLoadedModel(LoadedModel* loadedModel) { delete loadedModel; }
const ModelDesc& NeuralNet::getModelDesc(const LoadedModel* loadedModel) { return loadedModel->modelDesc; }

// Global ------------------------------------------------------------------------------------------

void NeuralNet::globalInitialize() {}
void NeuralNet::globalCleanup() {}

void NeuralNet::printDevices() {
  int count = 0;
  if(kb_device_count(&count) != 0) {
    cout << "B200 backend: " << kb_last_error() << endl;
    return;
  }
  for(int i = 0; i < count; i++) {
    char name[256];
    if(kb_device_name(i, name, sizeof(name)) == 0)
      cout << "Found GPU device " << i << ": " << name << endl;
  }
}

// Context -----------------------------------------------------------------------------------------

struct ComputeContext {
  int nnXLen;
  int nnYLen;
  int precision;  // KB_PRECISION_*
  kb_model* model;
  ~ComputeContext() { kb_model_destroy(model); }
};

ComputeContext* NeuralNet::createComputeContext(
  const std::vector<int>& gpuIdxs, Logger* logger, int nnXLen, int nnYLen, const string& homeDataDirOverride,
  enabled_t useFP16Mode, const LoadedModel* loadedModel, ConfigParser& cfg) {
  (void)gpuIdxs;
  (void)logger;
  (void)homeDataDirOverride;  // no tuning files or plan caches: the tile configuration is compiled in
  auto context = std::make_unique<ComputeContext>();
  context->nnXLen = nnXLen;
  context->nnYLen = nnYLen;
  context->model = nullptr;
  if(useFP16Mode == enabled_t::False) {
    context->precision = KB_PRECISION_FP32;
  }
  else {
    string prec = "fp16";
    if(cfg.contains("cudaPrecision"))
      prec = Global::toLower(cfg.getString("cudaPrecision"));
    else if(const char* e = std::getenv("KATAB200_PRECISION"))
      prec = Global::toLower(string(e));
    if(prec == "fp16") context->precision = KB_PRECISION_FP16;
    else if(prec == "bf16") context->precision = KB_PRECISION_BF16;
    else if(prec == "fp32") context->precision = KB_PRECISION_FP32;
    else throw StringError("B200 backend: cudaPrecision must be fp16, bf16 or fp32, got " + prec);
  }
  // The device library works on the flattened model; built once per context and shared by all handles.
  std::vector<uint32_t> blob = kbhost::modelDescToBlob(loadedModel->modelDesc, loadedModel->ext.empty() ? nullptr : &loadedModel->ext);
  check(kb_model_create(blob.data(), blob.size() * sizeof(uint32_t), &context->model), "kb_model_create");
  return context.release();
}

void NeuralNet::freeComputeContext(ComputeContext* computeContext) { delete computeContext; }

// Handle ------------------------------------------------------------------------------------------

// Host-side stage timers of getOutput (environment KATAB200_TIMING=1): where a server thread's wall time goes.  "waiting"
// is the time between the return of one getOutput and the entry of the next, i.e. the NNEvaluator queue filling up.
struct StageTimers {
  typedef std::chrono::steady_clock Clock;
  bool on = false;
  int serverThreadIdx = 0, gpuIdx = 0;
  long long calls = 0, rows = 0;
  double stageS = 0.0, deviceS = 0.0, unpackS = 0.0, waitingS = 0.0;
  Clock::time_point lastReturn;
  bool hasLast = false;
  static double since(Clock::time_point t0, Clock::time_point t1) { return std::chrono::duration<double>(t1 - t0).count(); }
  void report() const {
    if(!on || calls == 0) return;
    std::fprintf(
      stderr,
      "B200 backend timing: server thread %d (GPU %d): %lld getOutput calls, %lld rows (%.1f per call); staging rows %.3f s, "
      "kb_forward_host %.3f s, unpacking %.3f s, waiting for the next batch %.3f s\n",
      serverThreadIdx, gpuIdx, calls, rows, (double)rows / (double)calls, stageS, deviceS, unpackS, waitingS);
  }
};

struct ComputeHandle {
  kb_handle* handle = nullptr;
  kbhost::NetDims dims;
  int precision = KB_PRECISION_FP32;
  int maxBatchSize = 0;
  bool inputsUseNHWC = true;
  StageTimers timers;
  ~ComputeHandle() {
    timers.report();
    kb_handle_destroy(handle);
  }
};

ComputeHandle* NeuralNet::createComputeHandle(
  ComputeContext* context, const LoadedModel* loadedModel, Logger* logger, int maxBatchSize, bool requireExactNNLen,
  bool inputsUseNHWC, int gpuIdxForThisThread, int serverThreadIdx) {
  auto handle = std::make_unique<ComputeHandle>();
  handle->dims = kbhost::makeNetDims(loadedModel->modelDesc, context->nnXLen, context->nnYLen);
  handle->precision = context->precision;
  handle->maxBatchSize = maxBatchSize;
  handle->inputsUseNHWC = inputsUseNHWC;
  {
    const char* e = std::getenv("KATAB200_TIMING");
    handle->timers.on = e != NULL && std::atoi(e) != 0;
    handle->timers.serverThreadIdx = serverThreadIdx;
    handle->timers.gpuIdx = gpuIdxForThisThread;
  }
  check(
    kb_handle_create(
      context->model, gpuIdxForThisThread, maxBatchSize, context->nnXLen, context->nnYLen, context->precision,
      requireExactNNLen ? 1 : 0, &handle->handle),
    "kb_handle_create");
  if(logger != NULL) {
    const char* precName = context->precision == KB_PRECISION_FP32 ? "fp32" : (context->precision == KB_PRECISION_FP16 ? "fp16" : "bf16");
    logger->write(
      "B200 backend thread " + Global::intToString(serverThreadIdx) + ": GPU " + Global::intToString(gpuIdxForThisThread) +
      " precision " + precName + " NHWC");
    logger->write("B200 backend thread " + Global::intToString(serverThreadIdx) + ": Model version " + Global::intToString(loadedModel->modelDesc.modelVersion));
    logger->write(
      "B200 backend thread " + Global::intToString(serverThreadIdx) + ": Model name: " + loadedModel->modelDesc.name + " (" +
      loadedModel->modelDesc.getShortInfoString() + ")");
  }
  return handle.release();
}

void NeuralNet::freeComputeHandle(ComputeHandle* gpuHandle) { delete gpuHandle; }

bool NeuralNet::isUsingFP16(const ComputeHandle* handle) { return handle->precision != KB_PRECISION_FP32; }

bool NeuralNet::setIsWarmup(const ComputeHandle* handle, bool isWarmup) {
  (void)handle;
  (void)isWarmup;
  return false;
}

// Input buffers -----------------------------------------------------------------------------------
// Created before the handle and without a device bound (nneval.cpp:359 vs 559), so the page-locked
// staging memory comes from kb_host_alloc, which needs no current device.

struct InputBuffers {
  int maxBatchSize = 0;
  size_t singleInputElts = 0;
  size_t singleGlobalElts = 0;
  size_t singleMetaElts = 0;  // 0 for nets without an SGF metadata encoder
  size_t S = 0;
  int policyC = 0, valueC = 0, scoreValueC = 0;
  float* spatial = nullptr;
  float* global = nullptr;
  float* meta = nullptr;
  int32_t* symmetry = nullptr;
  float* policy = nullptr;
  float* policyPass = nullptr;
  float* value = nullptr;
  float* scoreValue = nullptr;
  float* ownership = nullptr;
  std::vector<float> scratchRow;
  std::vector<void*> owned;

  template <typename T>
  T* pinned(size_t count) {
    void* p = nullptr;
    check(kb_host_alloc(std::max<size_t>(count, 4) * sizeof(T), &p), "kb_host_alloc");
    owned.push_back(p);
    return static_cast<T*>(p);
  }
  ~InputBuffers() {
    for(void* p : owned) kb_host_free(p);
  }
};

InputBuffers* NeuralNet::createInputBuffers(const LoadedModel* loadedModel, int maxBatchSize, int nnXLen, int nnYLen) {
  const ModelDesc& m = loadedModel->modelDesc;
  auto b = std::make_unique<InputBuffers>();
  b->maxBatchSize = maxBatchSize;
  b->S = (size_t)nnXLen * nnYLen;
  b->singleInputElts = b->S * m.numInputChannels;
  b->singleGlobalElts = (size_t)m.numInputGlobalChannels;
  b->policyC = m.numPolicyChannels;
  b->valueC = m.numValueChannels;
  b->scoreValueC = m.numScoreValueChannels;
  b->spatial = b->pinned<float>(b->singleInputElts * maxBatchSize);
  b->global = b->pinned<float>(b->singleGlobalElts * maxBatchSize);
  b->singleMetaElts = (size_t)m.numInputMetaChannels;
  if(b->singleMetaElts > 0) b->meta = b->pinned<float>(b->singleMetaElts * maxBatchSize);
  b->symmetry = b->pinned<int32_t>((size_t)maxBatchSize);
  b->policy = b->pinned<float>(b->S * b->policyC * maxBatchSize);
  b->policyPass = b->pinned<float>((size_t)b->policyC * maxBatchSize);
  b->value = b->pinned<float>((size_t)b->valueC * maxBatchSize);
  b->scoreValue = b->pinned<float>((size_t)b->scoreValueC * maxBatchSize);
  b->ownership = b->pinned<float>(b->S * maxBatchSize);
  b->scratchRow.resize(b->singleInputElts);
  return b.release();
}

void NeuralNet::freeInputBuffers(InputBuffers* buffers) { delete buffers; }

// getOutput ---------------------------------------------------------------------------------------

void NeuralNet::getOutput(
  ComputeHandle* h, InputBuffers* b, int numBatchEltsFilled, NNResultBuf** inputBufs, vector<NNOutput*>& outputs) {
  const int n = numBatchEltsFilled;
  if(n <= 0 || n > b->maxBatchSize || n > h->maxBatchSize || (int)outputs.size() != n)
    throw StringError("B200 backend: bad batch size in getOutput");
  const kbhost::NetDims& d = h->dims;
  const size_t S = b->S;
  const size_t C = (size_t)d.numSpatialFeatures;
  StageTimers& tm = h->timers;
  StageTimers::Clock::time_point t0, t1, t2;
  if(tm.on) {
    t0 = StageTimers::Clock::now();
    if(tm.hasLast) tm.waitingS += StageTimers::since(tm.lastReturn, t0);
  }

  // Stage rows.  The board symmetry is applied on the device (inputs) and inverted there (policy,
  // ownership), so rows are copied as they are; only an NCHW row needs a transposition here.
  for(int row = 0; row < n; row++) {
    const NNResultBuf* buf = inputBufs[row];
    // metadata rows exactly for nets with the encoder (eigenbackend.cpp:2462-2472)
    if((b->singleMetaElts > 0) != buf->hasRowMeta)
      throw StringError("B200 backend: SGF metadata rows must be given exactly for models with a metadata encoder");
    if(b->singleMetaElts > 0)
      std::memcpy(b->meta + b->singleMetaElts * row, buf->rowMetaBuf.data(), b->singleMetaElts * sizeof(float));
    float* dst = b->spatial + b->singleInputElts * row;
    const float* src = buf->rowSpatialBuf.data();
    if(h->inputsUseNHWC) {
      std::memcpy(dst, src, b->singleInputElts * sizeof(float));
    }
    else {
      for(size_t c = 0; c < C; c++)
        for(size_t s = 0; s < S; s++) dst[s * C + c] = src[c * S + s];
    }
    std::memcpy(b->global + b->singleGlobalElts * row, buf->rowGlobalBuf.data(), b->singleGlobalElts * sizeof(float));
    b->symmetry[row] = buf->symmetry;
  }

  if(tm.on) t1 = StageTimers::Clock::now();
  check(
    kb_forward_host_meta(
      h->handle, n, b->spatial, b->global, b->meta, b->symmetry, b->policy, b->policyPass, b->value, b->scoreValue, b->ownership),
    "kb_forward_host_meta");
  if(tm.on) t2 = StageTimers::Clock::now();

  // Unpack.  Symmetry was already inverted on the device, so unpackRow is called with identity symmetry.
  NNResultBuf identity;
  for(int row = 0; row < n; row++) {
    identity.symmetry = 0;
    identity.policyOptimism = inputBufs[row]->policyOptimism;
    kbhost::unpackRow(
      d, &identity, outputs[row], b->policy + S * d.numPolicyChannels * row, b->policyPass + (size_t)d.numPolicyChannels * row,
      b->value + (size_t)d.numValueChannels * row, b->scoreValue + (size_t)d.numScoreValueChannels * row, b->ownership + S * row);
  }
  if(tm.on) {
    const StageTimers::Clock::time_point t3 = StageTimers::Clock::now();
    tm.calls++; tm.rows += n;
    tm.stageS += StageTimers::since(t0, t1); tm.deviceS += StageTimers::since(t1, t2); tm.unpackS += StageTimers::since(t2, t3);
    tm.lastReturn = t3; tm.hasLast = true;
  }
}

// Layer tests -------------------------------------------------------------------------------------

static bool evalLayer(
  const std::vector<uint32_t>& blob, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC, int inC, int outC,
  const std::vector<float>& inputBuffer, const std::vector<float>* maskBuffer, std::vector<float>& outputBuffer) {
  std::vector<float> in = useNHWC ? inputBuffer : kbhost::nchwToNhwc(inputBuffer, batchSize, inC, nnYLen, nnXLen);
  std::vector<float> out((size_t)batchSize * nnXLen * nnYLen * outC);
  check(
    kb_eval_layer(
      blob.data(), blob.size() * sizeof(uint32_t), -1, useFP16 ? KB_PRECISION_FP16 : KB_PRECISION_FP32, batchSize, nnXLen, nnYLen,
      in.data(), maskBuffer ? maskBuffer->data() : nullptr, out.data()),
    "kb_eval_layer");
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
  const int c = desc->preBN.numChannels;
  return evalLayer(kbhost::ordinaryBlockToBlob(*desc), batchSize, nnXLen, nnYLen, useFP16, useNHWC, c, c, inputBuffer, &maskBuffer, outputBuffer);
}

bool NeuralNet::testEvaluateGlobalPoolingResidualBlock(
  const GlobalPoolingResidualBlockDesc* desc, int batchSize, int nnXLen, int nnYLen, bool useFP16, bool useNHWC,
  const std::vector<float>& inputBuffer, const std::vector<float>& maskBuffer, std::vector<float>& outputBuffer) {
  const int c = desc->preBN.numChannels;
  return evalLayer(kbhost::gpoolBlockToBlob(*desc), batchSize, nnXLen, nnYLen, useFP16, useNHWC, c, c, inputBuffer, &maskBuffer, outputBuffer);
}
