// One GPU replica of a network: device weights, activation buffers and the static launch list
// ("program") that one forward pass replays.  Mirrors the role of the reference CUDA backend's
// ComputeHandle + Model + Buffers (cpp/neuralnet/cudabackend.cpp:2852-3406) without its per-layer
// objects: the block graph is flattened once, at creation, into a list of fused launches.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "kb_kernels.cuh"
#include "kb_model.h"

namespace kb {

struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
void cudaCheck(cudaError_t e, const char* what);

// Counters of the device-side weight cache, summed over all devices: live entries, their bytes, uploads made and
// uploads avoided since the process started.
struct WeightCacheStats { int64_t entries, bytes, uploads, hits; };
WeightCacheStats weightCacheStats();

// One launch of the program.
struct Op {
  int cls = 0;                                   // index into Engine::classes (profiling bucket)
  double flops = 0.0, bytes = 0.0;               // algorithmic, per board (scaled by n when accounted)
  std::function<cudaError_t(cudaStream_t, const Geom&)> run;
  // tensor-core convolutions only: what the launch reads and writes, and its per-tile dependency record
  const ConvTcPlan* tcPlan = nullptr;
  Epilogue ep;
  const void* convIn = nullptr;   // input tensor, its row stride, weights and shape of the convolution
  const void* convW = nullptr;
  int convInStride = 0, convInC = 0, convOutC = 0, convK = 0;
  std::shared_ptr<ConvTcDeps> deps;
};

struct OpClass {
  std::string name;
  int64_t launches = 0;
  double ms = 0.0, flops = 0.0, bytes = 0.0;
};

class Engine {
 public:
  // Whole network.
  Engine(const Model& m, int device, int maxBatch, int X, int Y, int precision, bool requireExactNNLen);
  // Single layer (test entry points): blob holds one CONV / BN / block.
  Engine(const void* layerBlob, size_t nbytes, int device, int n, int X, int Y, int precision);
  ~Engine();
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  int precision() const { return dt_; }
  int launchesPerForward(int n) const {
    const int chunk = chunkBoards_ > 0 ? chunkBoards_ : n;
    return (int)ops_.size() * ((n + chunk - 1) / chunk);
  }

  // meta: [n][inMetaC] rows for nets with an SGF metadata encoder (must be non-NULL exactly for those nets)
  void uploadInputs(int n, const float* spatial, const float* global, const int32_t* symmetry, const float* meta = nullptr);
  int metaChannels() const { return inMetaC_; }
  void forwardResident(int n);
  void downloadOutputs(int n, float* policy, float* policyPass, float* value, float* scoreValue, float* ownership);
  float timeForwardResident(int n, int iters);
  void timeForwardSteps(int n, int steps, size_t flushBytes, float* msEach);
  void readTrunk(int n, float* out);

  // single-layer mode
  void evalLayer(const float* in, const float* mask, float* out);

  void profileEnable(bool on) { profiling_ = on; }
  void profileReset();
  int profileRead(OpClass* out, int cap);

  void sync();
  // Runs the wait self-test on this handle's stream and synchronises: throws CudaError like any timed-out wait.
  void selfTestWaitTimeout(unsigned long long limitNs);

 private:
  struct DevBuf { void* p = nullptr; size_t bytes = 0; };
  struct ConvDev {
    int kY = 1, kX = 1, inC = 0, outC = 0;  // inC as seen on the device (possibly zero-padded)
    int inCReal = 0;                         // the layer's own input channel count
    void* w = nullptr;
    bool tc = false;
    ConvTcPlan* plan = nullptr;
    const void* in = nullptr;
    int inStride = 0;
  };
  // The launch list of one batch size, captured into a CUDA graph the second time that size is run (the first run is
  // the eager warm-up); key = n * 2 + (symmetries given).  KB_NO_GRAPH=1 keeps every run eager.
  struct GraphEntry { int uses = 0; cudaGraphExec_t exec = nullptr; };
  std::map<int, GraphEntry> graphs_;
  bool graphsEnabled_ = true;
  int graphsInstantiated_ = 0;  // instantiated graphs (at most 64 batch sizes are captured; the others stay eager)
  void launchOpsEager(int n);

  // RMS norms of pre-norm transformer blocks folded into the convolutions around them: the producer of the residual
  // stream leaves per-row partial sums of squares, the consuming projection turns them into its row scale.
  float* rowSums_ = nullptr;   // [slot][rowsPadMax] partial sums of squares of the current stream's rows
  int rowSumsSlotsMax_ = 0;
  int rowSumsCur_ = -1;        // number of slots the current stream's producer filled, or -1: no sums available
  bool rowNormFold_ = false;
  void produceRowSums(Epilogue& ep, int k, int inC, int outC);

  struct BNDev { const float* scale = nullptr; const float* bias = nullptr; int act = 0; int C = 0; };

  // Read-only weights go through a process-wide cache per device, keyed by their contents: handles created from the
  // same model on the same device (the reference runs two server threads per GPU) share one copy, as the reference's
  // CPU backend shares one Model per name and hash (eigenbackend.cpp:2364-2392).  Entries are reference counted and
  // freed with their last handle.
  void* uploadShared(const void* host, size_t bytes);
  std::vector<void*> sharedWeights_;
  void* alloc(size_t bytes);                               // zero-initialised device memory
  void* scratch(const std::string& key, size_t bytes);     // named, reused across the plan
  float* uploadF32(const std::vector<float>& v);
  float* uploadF32Transposed(const std::vector<float>& w, int inC, int outC);
  void* uploadConvWeights(const std::vector<const ConvW*>& parts, int inCdev, bool tcLayout);
  ConvDev makeConv(const std::vector<const ConvW*>& parts, const void* in, int inStride, int inCdev);
  BNDev makeBN(const std::vector<const BNW*>& parts);
  int classId(const std::string& name);
  void addConvOp(const ConvDev& c, Epilogue ep, const std::string& tag);
  void addOp(const std::string& cls, double flops, double bytes, std::function<cudaError_t(cudaStream_t, const Geom&)> f);

  // Emits the launches of a block stack.  On entry `raw` holds the residual stream ([rows][C]) and, if the
  // first block wants it, `act` holds preBN+activation of it.  On exit `raw` is updated and `act` holds
  // tail-norm(raw) if `tail` is given.
  void emitStack(const std::vector<BlockW>& blocks, int C, void* raw, void* act, const BNW* tail, int depth, bool actValid);
  void emitBlock(const BlockW& b, int C, void* raw, void* act, const BNW* next, int depth);
  void emitHeads(const Model& m, const void* trunkAct);
  void runOps(int n);

  int device_ = 0, dt_ = DT_F32, X_ = 19, Y_ = 19, maxBatch_ = 1, rowsPadMax_ = 0;
  bool forceSimt_ = false;
  int chunkBoards_ = 0;   // boards per pass through the launch list (0 = whole batch)
  int boardOffset_ = 0;   // first board of the chunk being launched
  cudaStream_t stream_ = nullptr;
  std::vector<void*> allocations_;
  std::vector<size_t> allocationBytes_;
  // Per-tile dependencies between consecutive tensor-core convolutions (KB_TILE_DEPS): one counter per convolution
  // and 128-row tile, zeroed at the start of every pass through the launch list.
  bool tileDeps_ = false;
  int tileDepsMode_ = 0;
  uint32_t* tileCtr_ = nullptr;
  size_t tileCtrBytes_ = 0;
  void planTileDeps();
  // Multi-layer launches (KB_CHAIN: 0 off, 1 runs of 3x3 convolutions, 2 runs of any tensor-core convolutions): runs of
  // consecutive convolutions of the launch list become one persistent launch each.
  // Pairs (closing 1x1 of a nested bottleneck block, opening 1x1 of the next) as one launch (KB_FUSE_1X1=0: off).
  std::vector<ConvPostPrePlan*> postPrePlans_;
  void planPostPre();
  int chainMode_ = 0;
  std::vector<ConvChainPlan*> chainPlans_;
  void planChains();
  int allocationOf(const void* p) const;
  std::map<std::string, DevBuf> scratch_;
  std::vector<ConvTcPlan*> tcPlans_;
  std::vector<AttnTcPlan*> attnPlans_;
  std::vector<Op> ops_;
  std::vector<OpClass> classes_;
  bool profiling_ = false;
  std::vector<cudaEvent_t> events_;
  int* statusWord_ = nullptr;  // device
  int* statusHost_ = nullptr;  // pinned
  void* flushBuf_ = nullptr;
  size_t flushBytes_ = 0;

  // whole-network state
  int inC_ = 0, inCdev_ = 0, inGlobalC_ = 0, trunkC_ = 0, policyC_ = 0, valueC_ = 0, scoreValueC_ = 0;
  float* dMeta_ = nullptr;
  int inMetaC_ = 0;
  float *dSpatial_ = nullptr, *dGlobal_ = nullptr, *mask_ = nullptr, *maskSum_ = nullptr;
  int32_t* dSym_ = nullptr;
  bool haveSym_ = false;
  void* inputBuf_ = nullptr;
  void* trunkAct_ = nullptr;
  float *dPolicy_ = nullptr, *dPolicyPass_ = nullptr, *dValue_ = nullptr, *dScore_ = nullptr, *dOwnership_ = nullptr;

  // single-layer state
  int layerN_ = 0, layerInC_ = 0, layerOutC_ = 0;
  float *layerIn_ = nullptr, *layerMaskIn_ = nullptr, *layerOut_ = nullptr;
  bool layerNeedsMask_ = false;
};

}  // namespace kb
