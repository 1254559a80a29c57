// Engine: flattens a kb::Model into a static list of fused launches and replays it.
//
// Fusion scheme.  Every convolution reads an ALREADY ACTIVATED tensor and its epilogue produces what its
// consumers need: the updated residual stream (accumulator + residual, stored raw) and/or the NEXT
// layer's batch-norm + activation + mask of that value.  So the reference's separate passes
// (BatchNormLayer::apply before every conv, the residual add, addNCBiasInplace; eigenbackend.cpp:1026-1303)
// disappear into the conv kernels; what remains besides convolutions is the gpool reduction, a few
// per-board matmuls and one elementwise pass per gpool block.
#include "kb_engine.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

namespace kb {

void cudaCheck(cudaError_t e, const char* what) {
  if(e != cudaSuccess) throw CudaError(std::string(what) + ": " + cudaGetErrorString(e));
}

static bool isConvBlock(const BlockW& b) { return b.kind == BLOCK_ORDINARY || b.kind == BLOCK_GPOOL || b.kind == BLOCK_NESTED; }

// host fp32 -> device dtype conversion
static void convertTo(int dt, const std::vector<float>& src, std::vector<uint8_t>& dst) {
  dst.resize(src.size() * dtypeSize(dt));
  if(dt == DT_F32) std::memcpy(dst.data(), src.data(), src.size() * 4);
  else if(dt == DT_F16) {
    __half* o = reinterpret_cast<__half*>(dst.data());
    for(size_t i = 0; i < src.size(); i++) o[i] = __float2half_rn(src[i]);
  }
  else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(dst.data());
    for(size_t i = 0; i < src.size(); i++) o[i] = __float2bfloat16_rn(src[i]);
  }
}

// ---------------------------------------------------------------------------------------------

void* Engine::alloc(size_t bytes) {
  void* p = nullptr;
  if(bytes == 0) bytes = 16;
  cudaCheck(cudaMalloc(&p, bytes), "cudaMalloc");
  allocations_.push_back(p);
  allocationBytes_.push_back(bytes);
  cudaCheck(cudaMemsetAsync(p, 0, bytes, stream_), "cudaMemset");
  return p;
}

// ---------------------------------------------------------------------------------------------
// Weight cache

namespace {
struct WeightKey {
  int device; size_t bytes; uint64_t h1, h2;
  bool operator<(const WeightKey& o) const {
    if(device != o.device) return device < o.device;
    if(bytes != o.bytes) return bytes < o.bytes;
    if(h1 != o.h1) return h1 < o.h1;
    return h2 < o.h2;
  }
};
struct WeightEntry { void* p; int refs; };
std::mutex g_weightMu;
std::map<WeightKey, WeightEntry> g_weights;
std::map<const void*, WeightKey> g_weightOf;
int64_t g_weightUploads = 0, g_weightHits = 0;

// two independent 64-bit hashes of the bytes (FNV-1a and a multiply-rotate mix): 128 bits identify the contents
void hashBytes(const void* data, size_t n, uint64_t& h1, uint64_t& h2) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  h1 = 1469598103934665603ull; h2 = 0x9E3779B97F4A7C15ull ^ (uint64_t)n;
  size_t i = 0;
  for(; i + 8 <= n; i += 8) {
    uint64_t w;
    std::memcpy(&w, p + i, 8);
    h1 = (h1 ^ w) * 1099511628211ull;
    h2 = (h2 + w) * 0xC2B2AE3D27D4EB4Full;
    h2 = (h2 << 31) | (h2 >> 33);
  }
  for(; i < n; i++) { h1 = (h1 ^ p[i]) * 1099511628211ull; h2 = (h2 + p[i]) * 0x165667B19E3779F9ull; }
}
}  // namespace

WeightCacheStats weightCacheStats() {
  std::lock_guard<std::mutex> lock(g_weightMu);
  WeightCacheStats s = {0, 0, g_weightUploads, g_weightHits};
  for(const auto& kv : g_weights) { s.entries++; s.bytes += (int64_t)kv.first.bytes; }
  return s;
}

void* Engine::uploadShared(const void* host, size_t bytes) {
  static const bool enabled = getenv("KB_NO_WEIGHT_CACHE") == nullptr;
  if(bytes == 0) return alloc(16);
  WeightKey key;
  key.device = device_; key.bytes = bytes;
  hashBytes(host, bytes, key.h1, key.h2);
  std::lock_guard<std::mutex> lock(g_weightMu);
  if(enabled) {
    auto it = g_weights.find(key);
    if(it != g_weights.end()) {
      it->second.refs++;
      g_weightHits++;
      sharedWeights_.push_back(it->second.p);
      return it->second.p;
    }
  }
  void* p = nullptr;
  cudaCheck(cudaMalloc(&p, bytes), "cudaMalloc (weights)");
  cudaError_t e = cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, stream_);
  if(e == cudaSuccess) e = cudaStreamSynchronize(stream_);
  if(e != cudaSuccess) { cudaFree(p); cudaCheck(e, "upload weights"); }
  g_weightUploads++;
  if(!enabled) {
    // not shared: owned by this handle like any other allocation
    allocations_.push_back(p);
    allocationBytes_.push_back(bytes);
    return p;
  }
  g_weights[key] = WeightEntry{p, 1};
  g_weightOf[p] = key;
  sharedWeights_.push_back(p);
  return p;
}

void* Engine::scratch(const std::string& key, size_t bytes) {
  auto it = scratch_.find(key);
  if(it != scratch_.end()) {
    if(it->second.bytes < bytes) throw std::runtime_error("internal: scratch buffer " + key + " requested with two sizes");
    return it->second.p;
  }
  DevBuf b;
  b.p = alloc(bytes);
  b.bytes = bytes;
  scratch_[key] = b;
  return b.p;
}

float* Engine::uploadF32(const std::vector<float>& v) {
  return static_cast<float*>(uploadShared(v.data(), v.size() * sizeof(float)));
}

// [in][out] matmul weights stored output-major ([out][in]) for the fused per-board kernels
float* Engine::uploadF32Transposed(const std::vector<float>& w, int inC, int outC) {
  std::vector<float> t((size_t)inC * outC);
  for(int ic = 0; ic < inC; ic++)
    for(int oc = 0; oc < outC; oc++) t[(size_t)oc * inC + ic] = w[(size_t)ic * outC + oc];
  return uploadF32(t);
}

void* Engine::uploadConvWeights(const std::vector<const ConvW*>& parts, int inCdev, bool tcLayout) {
  const int kY = parts[0]->kY, kX = parts[0]->kX, inC = parts[0]->inC;
  int outC = 0;
  for(const ConvW* p : parts) {
    if(p->kY != kY || p->kX != kX || p->inC != inC) throw std::runtime_error("internal: merged convolutions differ in shape");
    outC += p->outC;
  }
  const int taps = kY * kX;
  std::vector<float> packed((size_t)taps * inCdev * outC, 0.0f);
  int oc0 = 0;
  for(const ConvW* p : parts) {
    for(int oc = 0; oc < p->outC; oc++)
      for(int ic = 0; ic < inC; ic++)
        for(int y = 0; y < kY; y++)
          for(int x = 0; x < kX; x++) {
            const float v = p->w[(((size_t)oc * inC + ic) * kY + y) * kX + x];
            const int tap = y * kX + x;
            const size_t dst = tcLayout ? ((size_t)tap * outC + (oc0 + oc)) * inCdev + ic
                                        : ((size_t)tap * inCdev + ic) * outC + (oc0 + oc);
            packed[dst] = v;
          }
    oc0 += p->outC;
  }
  std::vector<uint8_t> bytes;
  convertTo(dt_, packed, bytes);
  return uploadShared(bytes.data(), bytes.size());
}

Engine::ConvDev Engine::makeConv(const std::vector<const ConvW*>& parts, const void* in, int inStride, int inCdev) {
  ConvDev c;
  c.kY = parts[0]->kY; c.kX = parts[0]->kX; c.inC = inCdev; c.inCReal = parts[0]->inC;
  c.outC = 0;
  bool aligned = true;
  for(const ConvW* p : parts) { c.outC += p->outC; if(p->outC % 16) aligned = false; }
  c.in = in; c.inStride = inStride;
  c.tc = !forceSimt_ && aligned && convTcEligible(dt_, inCdev, c.outC, c.kY, c.kX) && (inStride % 8) == 0;
  c.w = uploadConvWeights(parts, inCdev, c.tc);
  if(c.tc) {
    c.plan = convTcCreate(dt_, in, inStride, inCdev, c.w, c.outC, c.kY, c.kX, X_, Y_, rowsPadMax_);
    if(!c.plan) throw std::runtime_error("failed to create the tensor-core convolution plan (TMA descriptor encoding)");
    tcPlans_.push_back(c.plan);
  }
  return c;
}

Engine::BNDev Engine::makeBN(const std::vector<const BNW*>& parts) {
  std::vector<float> s, b;
  BNDev d;
  d.act = parts[0]->act;
  for(const BNW* p : parts) {
    if(p->act != d.act) throw std::runtime_error("internal: merged norms differ in activation");
    s.insert(s.end(), p->scale.begin(), p->scale.end());
    b.insert(b.end(), p->bias.begin(), p->bias.end());
  }
  d.C = (int)s.size();
  d.scale = uploadF32(s);
  d.bias = uploadF32(b);
  return d;
}

int Engine::classId(const std::string& name) {
  for(size_t i = 0; i < classes_.size(); i++)
    if(classes_[i].name == name) return (int)i;
  OpClass c;
  c.name = name;
  classes_.push_back(c);
  return (int)classes_.size() - 1;
}

void Engine::addOp(const std::string& cls, double flops, double bytes, std::function<cudaError_t(cudaStream_t, const Geom&)> f) {
  Op op;
  op.cls = classId(cls);
  op.flops = flops;
  op.bytes = bytes;
  op.run = std::move(f);
  ops_.push_back(std::move(op));
}

void Engine::addConvOp(const ConvDev& c, Epilogue ep, const std::string& tag) {
  ep.mask = mask_;
  const double S = (double)X_ * Y_;
  const double es = (double)dtypeSize(dt_);
  double flops = 2.0 * c.kY * c.kX * c.inCReal * c.outC * S;
  double bytes = S * c.inCReal * es;
  if(ep.residual) bytes += S * c.outC * es;
  if(ep.outRaw) bytes += S * (ep.rawC1 - ep.rawC0) * es;
  if(ep.outAct) bytes += S * (ep.actC1 - ep.actC0) * es / (ep.act == KB_ACT_SWIGLU_PAIRS ? 2 : 1);
  std::string name = "conv" + std::to_string(c.kY) + "x" + std::to_string(c.kX) + " " + std::to_string(c.inCReal) + "->" +
                     std::to_string(c.outC) + (c.tc ? " tcgen05" : " simt") + (tag.empty() ? "" : " " + tag);
  const int dt = dt_;
  int* status = statusWord_;
  if(c.tc) {
    if(!convTcSetEpilogue(c.plan, ep)) throw std::runtime_error("tensor-core convolution: shared memory budget exceeded");
    if(ep.sumsqOut) {
      // the producer's slot count follows from the epilogue variant just chosen
      const int slots = convTcPlanRowSumSlots(c.plan);
      if(slots < 1 || slots > rowSumsSlotsMax_) throw std::runtime_error("internal: row-sum slots of a convolution exceed the buffer");
      rowSumsCur_ = slots;
    }
    const ConvTcPlan* plan = c.plan;
    std::shared_ptr<ConvTcDeps> deps = std::make_shared<ConvTcDeps>();
    addOp(name, flops, bytes, [plan, ep, status, deps](cudaStream_t st, const Geom& g) { return launchConvTc(st, plan, g, ep, status, deps.get()); });
    ops_.back().tcPlan = plan;
    ops_.back().ep = ep;
    ops_.back().deps = deps;
    ops_.back().convIn = c.in; ops_.back().convW = c.w; ops_.back().convInStride = c.inStride;
    ops_.back().convInC = c.inC; ops_.back().convOutC = c.outC; ops_.back().convK = c.kY;
  }
  else {
    ConvDev cc = c;
    addOp(name, flops, bytes, [cc, ep, dt](cudaStream_t st, const Geom& g) {
      return launchConvSimt(st, dt, cc.in, cc.inStride, cc.inC, cc.w, cc.outC, cc.kY, cc.kX, g, ep);
    });
  }
}

// A matmul (or several sharing their input, concatenated along the output channels) as a 1x1 convolution:
// MatMulW weights are [ic][oc], ConvW weights [oc][ic].
static ConvW matmulsAsConv(const std::vector<const MatMulW*>& parts) {
  ConvW c;
  c.kY = 1; c.kX = 1; c.inC = parts[0]->inC; c.outC = 0;
  for(const MatMulW* m : parts) {
    if(m->inC != c.inC) throw std::runtime_error("internal: merged matmuls differ in input width");
    c.outC += m->outC;
  }
  c.w.resize((size_t)c.inC * c.outC);
  int oc0 = 0;
  for(const MatMulW* m : parts) {
    for(int ic = 0; ic < m->inC; ic++)
      for(int oc = 0; oc < m->outC; oc++) c.w[(size_t)(oc0 + oc) * c.inC + ic] = m->w[(size_t)ic * m->outC + oc];
    oc0 += m->outC;
  }
  return c;
}

// conv(rmsnorm(x)) = rowScale * conv'(x) with the norm's gain folded into the weights: w'[oc][ic] = w[oc][ic] * gamma[ic].
static void foldGain(ConvW& c, const std::vector<float>& gamma) {
  if((int)gamma.size() != c.inC || c.kY != 1 || c.kX != 1) throw std::runtime_error("internal: cannot fold a norm gain into this convolution");
  for(int oc = 0; oc < c.outC; oc++)
    for(int ic = 0; ic < c.inC; ic++) c.w[(size_t)oc * c.inC + ic] *= gamma[ic];
}

// The same tables in factored form for the tensor-core attention kernel: the angle of pair p at (x,y) is an x part plus a
// y part (learnable: x*fx + y*fy; fixed theta: the first half of the pairs turns with y, the second with x), so
// (cos, sin) of the parts, [tableHeads][pairs][X] and [tableHeads][pairs][Y] as interleaved floats, give every angle by
// the addition theorem.
static void ropeFactorTables(const BlockW& b, int X, int Y, std::vector<float>& tx, std::vector<float>& ty, int& tableHeads) {
  const int pairs = b.qDim / 2;
  tableHeads = b.learnableRope ? b.kvHeads : 1;
  tx.assign((size_t)tableHeads * pairs * X * 2, 0.0f);
  ty.assign((size_t)tableHeads * pairs * Y * 2, 0.0f);
  const int pairsPerDim = pairs / 2, dimHalf = b.qDim / 2;
  for(int h = 0; h < tableHeads; h++)
    for(int p = 0; p < pairs; p++) {
      float fx, fy;
      if(b.learnableRope) { fx = b.ropeFreqs[(h * pairs + p) * 2 + 0]; fy = b.ropeFreqs[(h * pairs + p) * 2 + 1]; }
      else if(p < pairsPerDim) { fx = 0.0f; fy = 1.0f / powf(b.ropeTheta, (float)(2 * p) / (float)dimHalf); }
      else { fx = 1.0f / powf(b.ropeTheta, (float)(2 * (p - pairsPerDim)) / (float)dimHalf); fy = 0.0f; }
      for(int x = 0; x < X; x++) {
        const double a = (double)((float)x * fx);
        tx[(((size_t)h * pairs + p) * X + x) * 2] = (float)cos(a); tx[(((size_t)h * pairs + p) * X + x) * 2 + 1] = (float)sin(a);
      }
      for(int y = 0; y < Y; y++) {
        const double a = (double)((float)y * fy);
        ty[(((size_t)h * pairs + p) * Y + y) * 2] = (float)cos(a); ty[(((size_t)h * pairs + p) * Y + y) * 2 + 1] = (float)sin(a);
      }
    }
}

// The merged FFN up|gate projection with its output channels interleaved in groups of 16 (16 up, their 16 gate), the
// order the tensor-core convolution's SwiGLU epilogue expects.
static ConvW upGateInterleaved(const MatMulW& up, const MatMulW& gate) {
  if(up.inC != gate.inC || up.outC != gate.outC || (up.outC % 16) != 0) throw std::runtime_error("internal: up/gate shapes cannot be interleaved");
  ConvW c;
  c.kY = 1; c.kX = 1; c.inC = up.inC; c.outC = 2 * up.outC;
  c.w.resize((size_t)c.inC * c.outC);
  for(int f = 0; f < up.outC; f++) {
    const int rowUp = (f / 16) * 32 + (f % 16), rowGate = rowUp + 16;
    for(int ic = 0; ic < up.inC; ic++) {
      c.w[(size_t)rowUp * c.inC + ic] = up.w[(size_t)ic * up.outC + f];
      c.w[(size_t)rowGate * c.inC + ic] = gate.w[(size_t)ic * gate.outC + f];
    }
  }
  return c;
}

// The rotary frequencies per output channel pair of the merged Q|K projection: entries 2i and 2i+1 are the x and y
// frequency of channel pair (2i, 2i+1), query heads first, then key heads (a query head uses the frequencies of its
// key-value head; fixed theta: the first half of a head's pairs turns with y, the second with x).
static std::vector<float> ropeChannelFreqs(const BlockW& b) {
  const int pairs = b.qDim / 2, pairsPerDim = pairs / 2, dimHalf = b.qDim / 2;
  std::vector<float> f((size_t)(b.heads + b.kvHeads) * b.qDim, 0.0f);
  for(int hh = 0; hh < b.heads + b.kvHeads; hh++) {
    const int kvh = hh < b.heads ? hh / (b.heads / b.kvHeads) : hh - b.heads;
    for(int p = 0; p < pairs; p++) {
      float fx, fy;
      if(b.learnableRope) { fx = b.ropeFreqs[(kvh * pairs + p) * 2 + 0]; fy = b.ropeFreqs[(kvh * pairs + p) * 2 + 1]; }
      else if(p < pairsPerDim) { fx = 0.0f; fy = 1.0f / powf(b.ropeTheta, (float)(2 * p) / (float)dimHalf); }
      else { fx = 1.0f / powf(b.ropeTheta, (float)(2 * (p - pairsPerDim)) / (float)dimHalf); fy = 0.0f; }
      f[((size_t)hh * pairs + p) * 2] = fx; f[((size_t)hh * pairs + p) * 2 + 1] = fy;
    }
  }
  return f;
}

// cos/sin tables of the rotary embedding, [tableHeads][pairs][S] (desc.cpp:1212-1275 computeRopeCosSin).
static void ropeTables(const BlockW& b, int X, int Y, std::vector<float>& cosT, std::vector<float>& sinT, int& tableHeads) {
  const int S = X * Y, pairs = b.qDim / 2;
  if(b.learnableRope) {
    tableHeads = b.kvHeads;
    cosT.assign((size_t)b.kvHeads * pairs * S, 0.0f); sinT.assign((size_t)b.kvHeads * pairs * S, 0.0f);
    for(int h = 0; h < b.kvHeads; h++)
      for(int p = 0; p < pairs; p++) {
        const float fx = b.ropeFreqs[(h * pairs + p) * 2 + 0], fy = b.ropeFreqs[(h * pairs + p) * 2 + 1];
        for(int y = 0; y < Y; y++)
          for(int x = 0; x < X; x++) {
            const float angle = (float)x * fx + (float)y * fy;
            const size_t idx = ((size_t)h * pairs + p) * S + y * X + x;
            cosT[idx] = cosf(angle); sinT[idx] = sinf(angle);
          }
      }
  }
  else {
    tableHeads = 1;
    const int pairsPerDim = pairs / 2, dimHalf = b.qDim / 2;
    cosT.assign((size_t)pairs * S, 0.0f); sinT.assign((size_t)pairs * S, 0.0f);
    for(int p = 0; p < pairs; p++)
      for(int y = 0; y < Y; y++)
        for(int x = 0; x < X; x++) {
          float angle;
          if(p < pairsPerDim) angle = (float)y * (1.0f / powf(b.ropeTheta, (float)(2 * p) / (float)dimHalf));
          else angle = (float)x * (1.0f / powf(b.ropeTheta, (float)(2 * (p - pairsPerDim)) / (float)dimHalf));
          const size_t idx = (size_t)p * S + y * X + x;
          cosT[idx] = cosf(angle); sinT[idx] = sinf(angle);
        }
  }
}

// ---------------------------------------------------------------------------------------------
// Block graph -> launches

// Called for a convolution whose raw output becomes the residual stream of a pre-norm transformer stack.
void Engine::produceRowSums(Epilogue& ep, int k, int inC, int outC) {
  rowSumsCur_ = -1;
  if(!rowNormFold_ || (k == 1 && !convTcRowNormEligible(dt_, inC, outC))) return;
  const int slots = convTcRowSumSlots(k, inC, outC);
  if(slots < 1 || slots > rowSumsSlotsMax_) return;
  ep.sumsqOut = rowSums_;
  ep.sumsqRowStride = rowsPadMax_;
  rowSumsCur_ = slots;
}

void Engine::emitStack(const std::vector<BlockW>& blocks, int C, void* raw, void* act, const BNW* tail, int depth, bool actValid) {
  for(size_t i = 0; i < blocks.size(); i++) {
    const BNW* next = tail;
    if(i + 1 < blocks.size()) next = isConvBlock(blocks[i + 1]) ? &blocks[i + 1].preBN : nullptr;
    if(isConvBlock(blocks[i]) && !actValid) {
      // the producer of `raw` could not apply this block's norm (first block after a layer of another kind)
      BNDev pb = makeBN({&blocks[i].preBN});
      const int dt = dt_;
      float* mask = mask_;
      addOp("norm+act", 0.0, 2.0 * X_ * Y_ * C * dtypeSize(dt_), [=](cudaStream_t st, const Geom& g) {
        return launchBnAct(st, dt, raw, C, pb.scale, pb.bias, pb.act, mask, dt, act, C, C, g);
      });
    }
    if(isConvBlock(blocks[i])) rowSumsCur_ = -1;  // its convolutions change the stream without recording row sums
    emitBlock(blocks[i], C, raw, act, next, depth);
    if(isConvBlock(blocks[i])) rowSumsCur_ = -1;
    actValid = next != nullptr;
  }
}

void Engine::emitBlock(const BlockW& b, int C, void* raw, void* act, const BNW* next, int depth) {
  const size_t es = dtypeSize(dt_);
  const std::string d = "_d" + std::to_string(depth);
  auto finishEp = [&](Epilogue& ep) {
    // residual add into the stream + (optionally) the next block's norm/activation
    ep.residual = raw; ep.resStride = C;
    ep.outRaw = raw; ep.rawStride = C; ep.rawC0 = 0; ep.rawC1 = C;
    if(next) {
      BNDev nb = makeBN({next});
      ep.outAct = act; ep.actStride = C; ep.actC0 = 0; ep.actC1 = C;
      ep.scale = nb.scale; ep.bias = nb.bias; ep.act = nb.act;
    }
  };

  if(b.kind == BLOCK_ORDINARY) {
    const int mid = b.conv1.outC;
    void* tmp = scratch("tmp" + d + "_c" + std::to_string(mid), (size_t)rowsPadMax_ * mid * es);
    ConvDev c1 = makeConv({&b.conv1}, act, C, C);
    BNDev mb = makeBN({&b.midBN});
    Epilogue e1;
    e1.outAct = tmp; e1.actStride = mid; e1.actC0 = 0; e1.actC1 = mid; e1.scale = mb.scale; e1.bias = mb.bias; e1.act = mb.act;
    addConvOp(c1, e1, "");
    ConvDev c2 = makeConv({&b.conv2}, tmp, mid, mid);
    Epilogue e2;
    finishEp(e2);
    addConvOp(c2, e2, "+res");
  }
  else if(b.kind == BLOCK_GPOOL) {
    const int reg = b.conv1.outC, gp = b.gpoolConv.outC;
    void* R = scratch("gpR" + d + "_c" + std::to_string(reg), (size_t)rowsPadMax_ * reg * es);
    void* G = scratch("gpG" + d + "_c" + std::to_string(gp), (size_t)rowsPadMax_ * gp * es);
    void* Ract = scratch("gpRact" + d + "_c" + std::to_string(reg), (size_t)rowsPadMax_ * reg * es);
    float* pooled = static_cast<float*>(scratch("gpPooled" + d + "_c" + std::to_string(gp), (size_t)maxBatch_ * 3 * gp * sizeof(float)));
    float* gbias = static_cast<float*>(scratch("gpBias" + d + "_c" + std::to_string(reg), (size_t)maxBatch_ * reg * sizeof(float)));
    BNDev gb = makeBN({&b.gpoolBN});
    if(b.conv1.kY == b.gpoolConv.kY && b.conv1.kX == b.gpoolConv.kX) {
      // regular and gpool convolutions read the same tensor: one launch, outputs split by channel range
      ConvDev c1 = makeConv({&b.conv1, &b.gpoolConv}, act, C, C);
      Epilogue e1;
      e1.outRaw = R; e1.rawStride = reg; e1.rawC0 = 0; e1.rawC1 = reg;
      e1.outAct = G; e1.actStride = gp; e1.actC0 = reg; e1.actC1 = reg + gp; e1.scale = gb.scale; e1.bias = gb.bias; e1.act = gb.act;
      addConvOp(c1, e1, "reg|gpool");
    }
    else {
      ConvDev cr = makeConv({&b.conv1}, act, C, C);
      Epilogue er;
      er.outRaw = R; er.rawStride = reg; er.rawC0 = 0; er.rawC1 = reg;
      addConvOp(cr, er, "reg");
      ConvDev cg = makeConv({&b.gpoolConv}, act, C, C);
      Epilogue eg;
      eg.outAct = G; eg.actStride = gp; eg.actC0 = 0; eg.actC1 = gp; eg.scale = gb.scale; eg.bias = gb.bias; eg.act = gb.act;
      addConvOp(cg, eg, "gpool");
    }
    const int dt = dt_;
    float* mask = mask_; float* maskSum = maskSum_;
    const double S = (double)X_ * Y_;
    float* wBias = uploadF32(b.gpoolToBias.w);
    BNDev mb = makeBN({&b.midBN});
    static const bool fuseMid = getenv("KB_NO_GPOOL_FUSE") == nullptr;
    if(fuseMid && gpoolMidEligible(dt, gp, gp, reg, reg, reg)) {
      // pooling, bias matmul and the bias + norm + activation pass as one launch (everything is per board)
      float* wBiasT = uploadF32Transposed(b.gpoolToBias.w, 3 * gp, reg);
      addOp("gpool+bias+norm+act", 2.0 * 3 * gp * reg, S * (gp + 2.0 * reg) * es, [=](cudaStream_t st, const Geom& g) {
        return launchGPoolMid(st, dt, G, gp, gp, R, reg, reg, wBiasT, mb.scale, mb.bias, mb.act, mask, maskSum, Ract, reg, g);
      });
    }
    else {
      addOp("gpool", 0.0, S * gp * es, [=](cudaStream_t st, const Geom& g) {
        return launchGPool(st, dt, G, gp, 0, gp, mask, maskSum, pooled, 0, g);
      });
      addOp("matmul small", 2.0 * 3 * gp * reg, 0.0, [=](cudaStream_t st, const Geom& g) {
        return launchMatMulSmall(st, pooled, 3 * gp, wBias, reg, nullptr, KB_ACT_IDENTITY, gbias, g.n);
      });
      addOp("bias+norm+act", 0.0, 2.0 * S * reg * es, [=](cudaStream_t st, const Geom& g) {
        return launchBiasBnAct(st, dt, R, reg, gbias, mb.scale, mb.bias, mb.act, mask, Ract, reg, reg, g);
      });
    }
    ConvDev c2 = makeConv({&b.conv2}, Ract, reg, reg);
    Epilogue e2;
    finishEp(e2);
    addConvOp(c2, e2, "+res");
  }
  else if(b.kind == BLOCK_NESTED) {
    const int mid = b.conv1.outC;
    const std::string d1 = "_d" + std::to_string(depth + 1);
    void* midRaw = scratch("nRaw" + d1 + "_c" + std::to_string(mid), (size_t)rowsPadMax_ * mid * es);
    void* midAct = scratch("nAct" + d1 + "_c" + std::to_string(mid), (size_t)rowsPadMax_ * mid * es);
    ConvDev c1 = makeConv({&b.conv1}, act, C, C);
    Epilogue e1;
    e1.outRaw = midRaw; e1.rawStride = mid; e1.rawC0 = 0; e1.rawC1 = mid;
    const bool innerConv = isConvBlock(b.inner[0]);
    if(innerConv) {
      BNDev ib = makeBN({&b.inner[0].preBN});
      e1.outAct = midAct; e1.actStride = mid; e1.actC0 = 0; e1.actC1 = mid; e1.scale = ib.scale; e1.bias = ib.bias; e1.act = ib.act;
    }
    addConvOp(c1, e1, "");
    emitStack(b.inner, mid, midRaw, midAct, &b.midBN, depth + 1, innerConv);
    ConvDev c2 = makeConv({&b.conv2}, midAct, mid, mid);
    Epilogue e2;
    finishEp(e2);
    addConvOp(c2, e2, "+res");
  }
  else if(b.kind == BLOCK_ATTN) {
    // eigenbackend.cpp:1307-1588: x += (Wo * attention(rope(Wq h), rope(Wk h), Wv h)) * mask, h = rmsnorm(x)
    const int dt = dt_;
    float* mask = mask_;
    const double S = (double)X_ * Y_;
    const int H = b.heads, Hkv = b.kvHeads, dq = b.qDim, dv = b.vDim;
    const int qC = H * dq, kC = Hkv * dq, vC = Hkv * dv, qkvC = qC + kC + vC, oC = H * dv;
    void* normed = scratch("tfNorm" + d + "_c" + std::to_string(C), (size_t)rowsPadMax_ * C * es);
    void* qkv = scratch("tfQKV" + d + "_c" + std::to_string(qkvC), (size_t)rowsPadMax_ * qkvC * es);
    void* attn = scratch("tfAttn" + d + "_c" + std::to_string(oC), (size_t)rowsPadMax_ * oC * es);
    float* gamma = uploadF32(b.preLN.weight);
    const float eps = b.preLN.eps;
    const bool attnTc = !forceSimt_ && attentionTcEligible(dt_, dq, dv, X_, Y_, qkvC, 0, qC, qC + kC, oC) &&
                        (b.relBias.empty() || (2 * b.relBiasY - 1) * (2 * b.relBiasX - 1) <= KB_ATTN_TC_REL_MAX);
    float* dCos = nullptr;
    float* dSin = nullptr;
    const float2* dRopeX = nullptr;
    const float2* dRopeY = nullptr;
    int tableHeads = 1;
    if(b.useRope && attnTc) {
      // rotation from factored tables: in the projection's epilogue where that variant exists, else by the attention
      // kernel itself, in shared memory
      std::vector<float> tx, ty;
      ropeFactorTables(b, X_, Y_, tx, ty, tableHeads);
      dRopeX = reinterpret_cast<const float2*>(uploadF32(tx));
      dRopeY = reinterpret_cast<const float2*>(uploadF32(ty));
    }
    const bool ropeFuseOff = getenv("KB_NO_ROPE_FUSE") != nullptr && atoi(getenv("KB_NO_ROPE_FUSE")) != 0;  // read per handle
    bool ropeInProjection = false;
    ConvW qkvW = matmulsAsConv({&b.q, &b.k, &b.v});
    Epilogue eq;
    eq.outRaw = qkv; eq.rawStride = qkvC; eq.rawC0 = 0; eq.rawC1 = qkvC;
    auto ropeEpilogue = [&](const ConvDev& cq) {
      if(!dRopeX || ropeFuseOff || !cq.tc || (dq % 2) != 0 || !convTcRopeEligible(dt_, C, qkvC, qC + kC)) return;
      eq.act = KB_ACT_ROPE_QK;
      eq.ropeFreq = uploadF32(ropeChannelFreqs(b));
      eq.ropeC1 = qC + kC;
      ropeInProjection = true;
    };
    if(rowSumsCur_ >= 0 && convTcRowNormEligible(dt_, C, qkvC)) {
      // the norm is folded into the projection: it reads the stream itself and scales its rows
      foldGain(qkvW, b.preLN.weight);
      ConvDev cq = makeConv({&qkvW}, raw, C, C);
      eq.rowSumsq = rowSums_; eq.rowSumsqSlots = rowSumsCur_; eq.sumsqRowStride = rowsPadMax_; eq.rowInvC = 1.0f / (float)C; eq.rowEps = eps;
      ropeEpilogue(cq);
      addConvOp(cq, eq, ropeInProjection ? "norm+qkv+rope" : "norm+qkv");
    }
    else {
      addOp("rmsnorm", 0.0, 2.0 * S * C * es, [=](cudaStream_t st, const Geom& g) {
        return launchRmsNorm(st, dt, raw, C, gamma, nullptr, eps, 0, mask, normed, C, C, g);
      });
      ConvDev cq = makeConv({&qkvW}, normed, C, C);
      ropeEpilogue(cq);
      addConvOp(cq, eq, ropeInProjection ? "qkv+rope" : "qkv");
    }
    if(ropeInProjection) { dRopeX = nullptr; dRopeY = nullptr; }
    else if(b.useRope && !attnTc) {
      std::vector<float> cosT, sinT;
      ropeTables(b, X_, Y_, cosT, sinT, tableHeads);
      dCos = uploadF32(cosT);
      dSin = uploadF32(sinT);
      {
        addOp("rope", 0.0, 2.0 * S * (qC + kC) * es, [=](cudaStream_t st, const Geom& g) {
          cudaError_t e = launchRope(st, dt, qkv, qkvC, 0, H, dq, dCos, dSin, tableHeads, g);
          if(e != cudaSuccess) return e;
          return launchRope(st, dt, qkv, qkvC, qC, Hkv, dq, dCos, dSin, tableHeads, g);
        });
      }
    }
    // optional learned relative-position bias (blob extension); both attention kernels take the table as it is
    const float* relBiasDev = nullptr;
    const int relY = b.relBiasY, relX = b.relBiasX;
    if(!b.relBias.empty()) {
      if(X_ > relX || Y_ > relY) throw std::runtime_error("attention block: board larger than the relative-position bias table");
      relBiasDev = uploadF32(b.relBias);
    }
    if(attnTc) {
      AttnTcPlan* ap = attentionTcCreate(dt_, qkv, qkvC, qkvC, rowsPadMax_);
      if(!ap) throw std::runtime_error("failed to create the tensor-core attention plan (TMA descriptor encoding)");
      attnPlans_.push_back(ap);
      int* status = statusWord_;
      // KB_ATTN_PIPE=0 (read when the handle is created): the one-CTA-per-(board, head) kernel also where the pipelined one applies
      const int pipelined = (getenv("KB_ATTN_PIPE") != nullptr && atoi(getenv("KB_ATTN_PIPE")) == 0) ? 0 : 1;
      addOp(dRopeX ? "attention tcgen05 +rope" : (pipelined ? "attention tcgen05 pipelined" : "attention tcgen05"), 2.0 * S * S * (dq + dv) * H, S * (qkvC + oC) * es, [=](cudaStream_t st, const Geom& g) {
        return launchAttentionTc(st, ap, 0, qC, qC + kC, H, Hkv, mask, attn, oC, g, status, dRopeX, dRopeY, tableHeads, relBiasDev, relY, relX, pipelined);
      });
    }
    else {
      if(!attentionFits(X_, Y_, dq, dv))
        throw std::runtime_error("attention block: a board of " + std::to_string(X_) + "x" + std::to_string(Y_) + " with head sizes " +
                                 std::to_string(dq) + "/" + std::to_string(dv) + " does not fit the attention kernel's shared memory");
      addOp("attention simt", 2.0 * S * S * (dq + dv) * H, S * (qkvC + oC) * es, [=](cudaStream_t st, const Geom& g) {
        return launchAttention(st, dt, qkv, qkvC, 0, qC, qC + kC, H, Hkv, dq, dv, mask, attn, oC, g, relBiasDev, relY, relX);
      });
    }
    ConvW outW = matmulsAsConv({&b.out});
    ConvDev co = makeConv({&outW}, attn, oC, oC);
    Epilogue eo;
    finishEp(eo);
    eo.resMask = 1;
    produceRowSums(eo, 1, oC, C);
    addConvOp(co, eo, "attn out +res");
  }
  else if(b.kind == BLOCK_FFN) {
    // eigenbackend.cpp:1592-1707: x += (W2 (silu(W1 h) * (Wg h))) * mask, h = rmsnorm(x)
    const int dt = dt_;
    float* mask = mask_;
    const double S = (double)X_ * Y_;
    const int F = b.ffnC;
    void* normed = scratch("tfNorm" + d + "_c" + std::to_string(C), (size_t)rowsPadMax_ * C * es);
    const bool needUp = forceSimt_ || !convTcSwigluEligible(dt_, C, F);
    void* up = needUp ? scratch("tfUp" + d + "_c" + std::to_string(2 * F), (size_t)rowsPadMax_ * 2 * F * es) : nullptr;
    void* hid = scratch("tfHid" + d + "_c" + std::to_string(F), (size_t)rowsPadMax_ * F * es);
    float* gamma = uploadF32(b.preLN.weight);
    const float eps = b.preLN.eps;
    const bool fuseSwiglu = !forceSimt_ && convTcSwigluEligible(dt_, C, F);
    const bool foldNorm = rowSumsCur_ >= 0 && convTcRowNormEligible(dt_, C, 2 * F);
    const void* ffnIn = foldNorm ? raw : normed;
    if(!foldNorm) {
      addOp("rmsnorm", 0.0, 2.0 * S * C * es, [=](cudaStream_t st, const Geom& g) {
        return launchRmsNorm(st, dt, raw, C, gamma, nullptr, eps, 0, mask, normed, C, C, g);
      });
    }
    ConvW upW = fuseSwiglu ? upGateInterleaved(b.linear1, b.gate) : matmulsAsConv({&b.linear1, &b.gate});
    if(foldNorm) foldGain(upW, b.preLN.weight);
    ConvDev cu = makeConv({&upW}, ffnIn, C, C);
    Epilogue eu;
    if(foldNorm) { eu.rowSumsq = rowSums_; eu.rowSumsqSlots = rowSumsCur_; eu.sumsqRowStride = rowsPadMax_; eu.rowInvC = 1.0f / (float)C; eu.rowEps = eps; }
    if(fuseSwiglu) {
      // one kernel: the projection's epilogue writes silu(up) * gate; the 2F-wide intermediate never reaches memory
      if(!cu.tc) throw std::runtime_error("internal: fused SwiGLU projection is not on the tensor-core path");
      eu.outAct = hid; eu.actStride = F; eu.actC0 = 0; eu.actC1 = 2 * F; eu.act = KB_ACT_SWIGLU_PAIRS;
      addConvOp(cu, eu, foldNorm ? "norm+ffn up|gate+swiglu" : "ffn up|gate+swiglu");
    }
    else {
      eu.outRaw = up; eu.rawStride = 2 * F; eu.rawC0 = 0; eu.rawC1 = 2 * F;
      addConvOp(cu, eu, foldNorm ? "norm+ffn up|gate" : "ffn up|gate");
      addOp("swiglu", 0.0, 3.0 * S * F * es, [=](cudaStream_t st, const Geom& g) { return launchSwiGLU(st, dt, up, 2 * F, hid, F, F, g); });
    }
    ConvW downW = matmulsAsConv({&b.linear2});
    ConvDev cd = makeConv({&downW}, hid, F, F);
    Epilogue ed;
    finishEp(ed);
    ed.resMask = 1;
    produceRowSums(ed, 1, F, C);
    addConvOp(cd, ed, "ffn down +res");
  }
  else {
    throw std::runtime_error("unknown block kind");
  }
}

void Engine::emitHeads(const Model& m, const void* trunkAct) {
  const size_t es = dtypeSize(dt_);
  const int P1 = m.p1Conv.outC, G1 = m.g1Conv.outC, V1 = m.v1Conv.outC, C = m.trunkC;
  const int dt = dt_;
  float* mask = mask_; float* maskSum = maskSum_;
  const double S = (double)X_ * Y_;
  void* Praw = scratch("headP", (size_t)rowsPadMax_ * P1 * es);
  void* Pact = scratch("headPact", (size_t)rowsPadMax_ * P1 * es);
  void* GV = scratch("headGV", (size_t)rowsPadMax_ * (G1 + V1) * es);
  float* gpooled = static_cast<float*>(scratch("headGPooled", (size_t)maxBatch_ * 3 * G1 * sizeof(float)));
  float* vpooled = static_cast<float*>(scratch("headVPooled", (size_t)maxBatch_ * 3 * V1 * sizeof(float)));
  float* pbias = static_cast<float*>(scratch("headPBias", (size_t)maxBatch_ * P1 * sizeof(float)));

  if(m.g1BN.act == m.v1BN.act) {
    // the three 1x1 convolutions that read the trunk run as one GEMM (reference: three cuDNN calls,
    // cudabackend.cpp:2603-2692, 2788-2846)
    ConvDev hc = makeConv({&m.p1Conv, &m.g1Conv, &m.v1Conv}, trunkAct, C, C);
    BNDev gv = makeBN({&m.g1BN, &m.v1BN});
    Epilogue e;
    e.outRaw = Praw; e.rawStride = P1; e.rawC0 = 0; e.rawC1 = P1;
    e.outAct = GV; e.actStride = G1 + V1; e.actC0 = P1; e.actC1 = P1 + G1 + V1; e.scale = gv.scale; e.bias = gv.bias; e.act = gv.act;
    addConvOp(hc, e, "heads p1|g1|v1");
  }
  else {
    ConvDev pc = makeConv({&m.p1Conv}, trunkAct, C, C);
    Epilogue ep;
    ep.outRaw = Praw; ep.rawStride = P1; ep.rawC0 = 0; ep.rawC1 = P1;
    addConvOp(pc, ep, "head p1");
    ConvDev gc = makeConv({&m.g1Conv}, trunkAct, C, C);
    BNDev gb = makeBN({&m.g1BN});
    Epilogue eg;
    eg.outAct = GV; eg.actStride = G1 + V1; eg.actC0 = 0; eg.actC1 = G1; eg.scale = gb.scale; eg.bias = gb.bias; eg.act = gb.act;
    addConvOp(gc, eg, "head g1");
    ConvDev vc = makeConv({&m.v1Conv}, trunkAct, C, C);
    BNDev vb = makeBN({&m.v1BN});
    Epilogue ev;
    ev.outAct = static_cast<uint8_t*>(GV) + (size_t)G1 * es; ev.actStride = G1 + V1; ev.actC0 = 0; ev.actC1 = V1;
    ev.scale = vb.scale; ev.bias = vb.bias; ev.act = vb.act;
    addConvOp(vc, ev, "head v1");
  }

  // weights of everything after the first convolutions
  float* wGB = uploadF32(m.gpoolToBias.w);
  float* dPass = dPolicyPass_;
  const int Pc = m.policyC;
  float* wPass = uploadF32(m.passMul.w);
  const int passH = m.hasPassMlp ? m.passMul.outC : 0;
  float* bPass = m.hasPassMlp ? uploadF32(m.passBias.b) : nullptr;
  float* wPass2 = m.hasPassMlp ? uploadF32(m.passMul2.w) : nullptr;
  const int passAct = m.passAct;
  BNDev pb = makeBN({&m.p1BN});
  const int V2 = m.v2Mul.outC, Vc = m.valueC, Sv = m.scoreValueC;
  float* wV2 = uploadF32(m.v2Mul.w); float* bV2 = uploadF32(m.v2Bias.b);
  float* wV3 = uploadF32(m.v3Mul.w); float* bV3 = uploadF32(m.v3Bias.b);
  float* wSV = uploadF32(m.sv3Mul.w); float* bSV = uploadF32(m.sv3Bias.b);
  float* dValue = dValue_; float* dScore = dScore_;
  const int v2Act = m.v2Act;
  // p2Conv [oc][ic][1][1] -> [ic][oc]; ownership conv [1][ic][1][1] -> [ic]
  std::vector<float> w2((size_t)P1 * Pc);
  for(int oc = 0; oc < Pc; oc++)
    for(int ic = 0; ic < P1; ic++) w2[(size_t)ic * Pc + oc] = m.p2Conv.w[(size_t)oc * P1 + ic];
  float* dW2 = uploadF32(w2);
  float* dWOwn = uploadF32(m.ownConv.w);
  float* dPolicy = dPolicy_; float* dOwn = dOwnership_;

  HeadsTailArgs ht;
  std::memset(&ht, 0, sizeof(ht));
  ht.pRaw = Praw; ht.gv = GV;
  ht.P1 = P1; ht.G1 = G1; ht.V1 = V1; ht.Pc = Pc; ht.Vc = Vc; ht.Sv = Sv; ht.V2 = V2; ht.passH = passH;
  ht.wGB = uploadF32Transposed(m.gpoolToBias.w, 3 * G1, P1);
  ht.wPass = uploadF32Transposed(m.passMul.w, 3 * G1, m.passMul.outC);
  ht.bPass = bPass; ht.passAct = passAct;
  ht.wPass2 = m.hasPassMlp ? uploadF32Transposed(m.passMul2.w, passH, Pc) : nullptr;
  ht.pScale = pb.scale; ht.pBias = pb.bias; ht.pAct = pb.act;
  ht.w2 = dW2; ht.wOwn = dWOwn;
  ht.wV2 = uploadF32Transposed(m.v2Mul.w, 3 * V1, V2); ht.bV2 = bV2; ht.v2Act = v2Act;
  ht.wV3 = uploadF32Transposed(m.v3Mul.w, V2, Vc); ht.bV3 = bV3;
  ht.wSV = uploadF32Transposed(m.sv3Mul.w, V2, Sv); ht.bSV = bSV;
  ht.mask = mask; ht.maskSum = maskSum;
  static const bool fuseTail = getenv("KB_NO_HEADS_FUSE") == nullptr;
  if(fuseTail && headsTailEligible(dt, ht)) {
    // poolings, policy bias, pass logits, value MLP, policy norm + activation + final convolution and the ownership
    // convolution: one launch, one CTA per board
    addOp("heads tail", 2.0 * S * (P1 * Pc + V1), S * (P1 + 2.0 * (G1 + V1)) * es + S * (Pc + 1) * 4.0, [=](cudaStream_t st, const Geom& g) {
      const size_t bo = (size_t)boardOffset_;
      HeadsTailArgs a = ht;
      a.symmetry = haveSym_ ? dSym_ + bo : nullptr;
      a.outPolicy = dPolicy + bo * g.S * Pc; a.outOwnership = dOwn + bo * g.S;
      a.outPass = dPass + bo * Pc; a.outValue = dValue + bo * Vc; a.outScore = dScore + bo * Sv;
      return launchHeadsTail(st, dt, a, g);
    });
    return;
  }

  addOp("gpool", 0.0, S * G1 * es, [=](cudaStream_t st, const Geom& g) {
    return launchGPool(st, dt, GV, G1 + V1, 0, G1, mask, maskSum, gpooled, 0, g);
  });
  addOp("gpool", 0.0, S * V1 * es, [=](cudaStream_t st, const Geom& g) {
    return launchGPool(st, dt, GV, G1 + V1, G1, V1, mask, maskSum, vpooled, 1, g);
  });
  addOp("matmul small", 2.0 * 3 * G1 * P1, 0.0, [=](cudaStream_t st, const Geom& g) {
    return launchMatMulSmall(st, gpooled, 3 * G1, wGB, P1, nullptr, KB_ACT_IDENTITY, pbias, g.n);
  });
  // pass logit (eigenbackend.cpp:2013-2022)
  if(m.hasPassMlp) {
    const int H = passH;
    float* hidden = static_cast<float*>(scratch("headPassHidden", (size_t)maxBatch_ * H * sizeof(float)));
    addOp("matmul small", 2.0 * 3 * G1 * H, 0.0, [=](cudaStream_t st, const Geom& g) {
      return launchMatMulSmall(st, gpooled, 3 * G1, wPass, H, bPass, passAct, hidden, g.n);
    });
    addOp("matmul small", 2.0 * H * Pc, 0.0, [=](cudaStream_t st, const Geom& g) {
      return launchMatMulSmall(st, hidden, H, wPass2, Pc, nullptr, KB_ACT_IDENTITY, dPass + (size_t)boardOffset_ * Pc, g.n);
    });
  }
  else {
    addOp("matmul small", 2.0 * 3 * G1 * Pc, 0.0, [=](cudaStream_t st, const Geom& g) {
      return launchMatMulSmall(st, gpooled, 3 * G1, wPass, Pc, nullptr, KB_ACT_IDENTITY, dPass + (size_t)boardOffset_ * Pc, g.n);
    });
  }
  addOp("bias+norm+act", 0.0, 2.0 * S * P1 * es, [=](cudaStream_t st, const Geom& g) {
    return launchBiasBnAct(st, dt, Praw, P1, pbias, pb.scale, pb.bias, pb.act, mask, Pact, P1, P1, g);
  });
  // value MLP (eigenbackend.cpp:2089-2099)
  float* v2 = static_cast<float*>(scratch("headV2", (size_t)maxBatch_ * V2 * sizeof(float)));
  addOp("matmul small", 2.0 * 3 * V1 * V2, 0.0, [=](cudaStream_t st, const Geom& g) {
    return launchMatMulSmall(st, vpooled, 3 * V1, wV2, V2, bV2, v2Act, v2, g.n);
  });
  addOp("matmul small", 2.0 * V2 * Vc, 0.0, [=](cudaStream_t st, const Geom& g) {
    return launchMatMulSmall(st, v2, V2, wV3, Vc, bV3, KB_ACT_IDENTITY, dValue + (size_t)boardOffset_ * Vc, g.n);
  });
  addOp("matmul small", 2.0 * V2 * Sv, 0.0, [=](cudaStream_t st, const Geom& g) {
    return launchMatMulSmall(st, v2, V2, wSV, Sv, bSV, KB_ACT_IDENTITY, dScore + (size_t)boardOffset_ * Sv, g.n);
  });
  addOp("head outputs", 2.0 * S * (P1 * Pc + V1), S * (P1 + V1) * es + S * (Pc + 1) * 4.0, [=](cudaStream_t st, const Geom& g) {
    const size_t bo = (size_t)boardOffset_;
    return launchHeadFinal(
      st, dt, Pact, P1, P1, dW2, Pc, GV, G1 + V1, G1, V1, dWOwn, haveSym_ ? dSym_ + bo : nullptr, dPolicy + bo * g.S * Pc, dOwn + bo * g.S, g);
  });
}

// ---------------------------------------------------------------------------------------------

static int pickDevice(int device) {
  int count = 0;
  cudaCheck(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
  if(count <= 0) throw CudaError("no CUDA device is available");
  if(device < 0) {
    cudaCheck(cudaGetDevice(&device), "cudaGetDevice");
  }
  if(device >= count) throw CudaError("device index " + std::to_string(device) + " is out of range (" + std::to_string(count) + " devices)");
  cudaCheck(cudaSetDevice(device), "cudaSetDevice");
  return device;
}

Engine::Engine(const Model& m, int device, int maxBatch, int X, int Y, int precision, bool requireExactNNLen) {
  (void)requireExactNNLen;  // masks are folded into epilogues that run anyway; exact-size boards need no special path
  if(maxBatch < 1 || maxBatch > 65536) throw std::runtime_error("maxBatch out of range");
  if(X < 2 || Y < 2 || X > 50 || Y > 50) throw std::runtime_error("board size out of range");
  if(precision != DT_F32 && precision != DT_F16 && precision != DT_BF16) throw std::runtime_error("unknown precision");
  device_ = pickDevice(device);
  dt_ = precision; X_ = X; Y_ = Y; maxBatch_ = maxBatch;
  forceSimt_ = getenv("KB_FORCE_SIMT") != nullptr && atoi(getenv("KB_FORCE_SIMT")) != 0;
  graphsEnabled_ = getenv("KB_NO_GRAPH") == nullptr;
  // 0: off; 1: 3x3 convolutions report their tiles (their epilogue warps have idle time to wait for the stores in);
  // 2: every tensor-core convolution reports
  tileDepsMode_ = getenv("KB_TILE_DEPS") != nullptr ? atoi(getenv("KB_TILE_DEPS")) : 0;
  tileDeps_ = tileDepsMode_ != 0;
  chunkBoards_ = 0;  // measured on B200: 128-board chunks 9.5 ms vs 8.1 ms for the whole batch of 256 (per-launch overhead wins)
  if(const char* e = getenv("KB_CHUNK_BOARDS")) chunkBoards_ = atoi(e);
  cudaCheck(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  const Geom gmax = makeGeom(X, Y, maxBatch);
  rowsPadMax_ = gmax.rowsPad;
  const size_t es = dtypeSize(dt_);
  const size_t S = (size_t)X * Y;
  inC_ = m.inC; inGlobalC_ = m.inGlobalC; trunkC_ = m.trunkC; policyC_ = m.policyC; valueC_ = m.valueC; scoreValueC_ = m.scoreValueC;
  statusWord_ = static_cast<int*>(alloc(sizeof(int)));
  cudaCheck(cudaHostAlloc(reinterpret_cast<void**>(&statusHost_), sizeof(int), cudaHostAllocDefault), "cudaHostAlloc");
  *statusHost_ = 0;

  const bool tcInit = !forceSimt_ && dt_ != DT_F32 && convTcEligible(dt_, 64, m.trunkC, m.initialConv.kY, m.initialConv.kX);
  inCdev_ = tcInit ? (m.inC + 63) / 64 * 64 : m.inC;

  dSpatial_ = static_cast<float*>(alloc((size_t)maxBatch * S * m.inC * sizeof(float)));
  dGlobal_ = static_cast<float*>(alloc((size_t)maxBatch * m.inGlobalC * sizeof(float)));
  inMetaC_ = m.inMetaC;
  if(inMetaC_ > 0) dMeta_ = static_cast<float*>(alloc((size_t)maxBatch * inMetaC_ * sizeof(float)));
  dSym_ = static_cast<int32_t*>(alloc((size_t)maxBatch * sizeof(int32_t)));
  mask_ = static_cast<float*>(alloc((size_t)rowsPadMax_ * sizeof(float)));
  maskSum_ = static_cast<float*>(alloc((size_t)maxBatch * sizeof(float)));
  inputBuf_ = alloc((size_t)rowsPadMax_ * inCdev_ * es);
  void* trunkRaw = alloc((size_t)rowsPadMax_ * m.trunkC * es);
  trunkAct_ = alloc((size_t)rowsPadMax_ * m.trunkC * es);
  float* gbias = static_cast<float*>(alloc((size_t)maxBatch * m.trunkC * sizeof(float)));
  dPolicy_ = static_cast<float*>(alloc((size_t)maxBatch * S * m.policyC * sizeof(float)));
  dPolicyPass_ = static_cast<float*>(alloc((size_t)maxBatch * m.policyC * sizeof(float)));
  dValue_ = static_cast<float*>(alloc((size_t)maxBatch * m.valueC * sizeof(float)));
  dScore_ = static_cast<float*>(alloc((size_t)maxBatch * m.scoreValueC * sizeof(float)));
  dOwnership_ = static_cast<float*>(alloc((size_t)maxBatch * S * sizeof(float)));

  // pre-norm transformer stacks on the tensor-core path: their norms are folded into the convolutions around them
  rowNormFold_ = !forceSimt_ && dt_ != DT_F32 && !isConvBlock(m.blocks[0]) && getenv("KB_NO_NORM_FOLD") == nullptr;
  if(rowNormFold_) {
    rowSumsSlotsMax_ = 32;
    rowSums_ = static_cast<float*>(alloc((size_t)rowSumsSlotsMax_ * rowsPadMax_ * sizeof(float)));
  }
  // input packing (symmetry, mask, maskSum)
  {
    const int dt = dt_, inC = inC_, inCdev = inCdev_;
    addOp("pack input", 0.0, (double)S * inC * 4.0 + (double)S * inCdev * es, [=](cudaStream_t st, const Geom& g) {
      const size_t bo = (size_t)boardOffset_;
      return launchPackInput(st, dt, dSpatial_ + bo * g.S * inC, haveSym_ ? dSym_ + bo : nullptr, inC, inputBuf_, inCdev, mask_, maskSum_, g);
    });
  }
  // global features -> per-board bias (eigenbackend.cpp:1913-1915)
  {
    float* wG = uploadF32(m.initialMatMul.w);
    const int inG = m.inGlobalC, tc = m.trunkC;
    addOp("matmul small", 2.0 * inG * tc, 0.0, [=](cudaStream_t st, const Geom& g) {
      return launchMatMulSmall(st, dGlobal_ + (size_t)boardOffset_ * inG, inG, wG, tc, nullptr, KB_ACT_IDENTITY, gbias, g.n);
    });
  }
  // SGF metadata encoder (eigenbackend.cpp:1801-1847, 1917-1920): a three-layer MLP on the metadata rows whose output is
  // added to the per-board bias
  if(m.inMetaC > 0) {
    const int inM = m.inMetaC, h1 = m.metaMul1.outC, h2 = m.metaMul2.outC, tc = m.trunkC, a1 = m.metaAct1, a2 = m.metaAct2;
    float* w1 = uploadF32(m.metaMul1.w); float* b1 = uploadF32(m.metaBias1.b);
    float* w2 = uploadF32(m.metaMul2.w); float* b2 = uploadF32(m.metaBias2.b);
    float* w3 = uploadF32(m.metaMul3.w);
    float* t1 = static_cast<float*>(alloc((size_t)maxBatch * h1 * sizeof(float)));
    float* t2 = static_cast<float*>(alloc((size_t)maxBatch * h2 * sizeof(float)));
    addOp("matmul small", 2.0 * inM * h1, 0.0, [=](cudaStream_t st, const Geom& g) {
      return launchMatMulSmall(st, dMeta_ + (size_t)boardOffset_ * inM, inM, w1, h1, b1, a1, t1, g.n);
    });
    addOp("matmul small", 2.0 * h1 * h2, 0.0, [=](cudaStream_t st, const Geom& g) { return launchMatMulSmall(st, t1, h1, w2, h2, b2, a2, t2, g.n); });
    addOp("matmul small", 2.0 * h2 * tc, 0.0, [=](cudaStream_t st, const Geom& g) {
      return launchMatMulSmall(st, t2, h2, w3, tc, nullptr, KB_ACT_IDENTITY, gbias, g.n, 1);
    });
  }
  // initial convolution + global bias, producing the stream and the first block's activated input
  {
    ConvDev c0 = makeConv({&m.initialConv}, inputBuf_, inCdev_, inCdev_);
    Epilogue e;
    e.biasNC = gbias;
    e.outRaw = trunkRaw; e.rawStride = m.trunkC; e.rawC0 = 0; e.rawC1 = m.trunkC;
    if(isConvBlock(m.blocks[0])) {
      BNDev b0 = makeBN({&m.blocks[0].preBN});
      e.outAct = trunkAct_; e.actStride = m.trunkC; e.actC0 = 0; e.actC1 = m.trunkC; e.scale = b0.scale; e.bias = b0.bias; e.act = b0.act;
    }
    else if(c0.tc && c0.kY == 3) {
      // the stem feeds a pre-norm transformer block: record the row sums of the stream it creates
      if((m.trunkC % 32) == 0) produceRowSums(e, c0.kY, c0.inC, m.trunkC);
    }
    addConvOp(c0, e, "initial");
  }
  emitStack(m.blocks, m.trunkC, trunkRaw, trunkAct_, m.normKind == 0 ? &m.tipBN : nullptr, 0, isConvBlock(m.blocks[0]));
  if(m.normKind != 0) {
    // RMSNorm trunk tip (eigenbackend.cpp:923-1022); only SiLU is applied as its activation, as in the reference
    float* gamma = uploadF32(m.tipRMS.gamma);
    float* beta = uploadF32(m.tipRMS.beta);
    const float eps = m.tipRMS.eps;
    const int silu = m.tipRMS.act == KB_ACT_SILU ? 1 : 0, spatial = m.tipRMS.spatial, C = m.trunkC, dt = dt_;
    float* boardScale = static_cast<float*>(alloc((size_t)maxBatch * sizeof(float)));
    void* tact = trunkAct_;
    float* mask = mask_;
    addOp("rmsnorm", 0.0, 2.0 * S * C * es, [=](cudaStream_t st, const Geom& g) {
      if(spatial) return launchSpatialRmsNorm(st, dt, trunkRaw, C, gamma, beta, eps, silu, mask, tact, C, C, boardScale, g);
      return launchRmsNorm(st, dt, trunkRaw, C, gamma, beta, eps, silu, mask, tact, C, C, g);
    });
  }
  emitHeads(m, trunkAct_);
  planPostPre();
  planChains();
  if(chainPlans_.empty()) planTileDeps();
  cudaCheck(cudaStreamSynchronize(stream_), "engine setup");
}

Engine::~Engine() {
  cudaSetDevice(device_);
  if(stream_) cudaStreamSynchronize(stream_);
  for(cudaEvent_t e : events_) cudaEventDestroy(e);
  for(ConvTcPlan* p : tcPlans_) convTcDestroy(p);
  for(AttnTcPlan* p : attnPlans_) attentionTcDestroy(p);
  for(ConvChainPlan* p : chainPlans_) convChainDestroy(p);
  for(ConvPostPrePlan* p : postPrePlans_) convPostPreDestroy(p);
  for(auto& kv : graphs_) if(kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  for(void* p : allocations_) cudaFree(p);
  {
    std::lock_guard<std::mutex> lock(g_weightMu);
    for(void* p : sharedWeights_) {
      auto ko = g_weightOf.find(p);
      if(ko == g_weightOf.end()) continue;
      auto it = g_weights.find(ko->second);
      if(it != g_weights.end() && --it->second.refs == 0) {
        cudaFree(it->second.p);
        g_weights.erase(it);
        g_weightOf.erase(ko);
      }
    }
  }
  if(statusHost_) cudaFreeHost(statusHost_);
  if(flushBuf_) cudaFree(flushBuf_);
  if(stream_) cudaStreamDestroy(stream_);
}

void Engine::sync() {
  cudaCheck(cudaStreamSynchronize(stream_), "stream synchronize");
  if(statusHost_ && *statusHost_ != 0) {
    int code = *statusHost_;
    *statusHost_ = 0;
    cudaMemsetAsync(statusWord_, 0, sizeof(int), stream_);
    throw CudaError("a device-side wait timed out (status " + std::to_string(code) + ": 101 producer, 102 MMA issuer, 103 epilogue of a tensor-core kernel, 199 wait self-test)");
  }
}

int Engine::allocationOf(const void* p) const {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  for(size_t i = 0; i < allocations_.size(); i++) {
    const uintptr_t b = reinterpret_cast<uintptr_t>(allocations_[i]);
    if(a >= b && a < b + allocationBytes_[i]) return (int)i;
  }
  return -1;
}

// Decides which tensor-core convolutions wait per tile on the convolution launched just before them instead of on
// its whole grid.  The launch itself (launchConvTc) additionally requires that the earlier convolution fills every SM.
// Reads are safe by construction (a tile reads rows of its own and the two neighbouring row tiles of whatever the
// earlier launch wrote, and waits for exactly those), and so are overwrites of buffers the earlier launch still
// reads (their readers are the same three tiles).  Excluded: inputs that kernels other than convolutions produce
// between the two (per-board bias, row sums), and a residual that the earlier launch itself wrote, because the
// epilogue fetches the residual ahead of the producer's wait.
// The closing 1x1 convolution of a nested bottleneck block writes the activated trunk tensor only for the opening 1x1
// convolution of the next block, launched right after it, to read it once.  Such a pair becomes one launch of
// convPostPreKernel, and the activated trunk tensor is not written at all.
void Engine::planPostPre() {
  const bool enabled = getenv("KB_FUSE_1X1") == nullptr || atoi(getenv("KB_FUSE_1X1")) != 0;
  if(!enabled || chunkBoards_ > 0 || layerN_ != 0 || forceSimt_) return;
  std::vector<Op> out;
  size_t i = 0;
  while(i < ops_.size()) {
    ConvPostPrePlan* plan = nullptr;
    if(i + 1 < ops_.size()) {
      const Op& A = ops_[i];
      const Op& B = ops_[i + 1];
      const Epilogue& ea = A.ep;
      const Epilogue& eb = B.ep;
      const bool shapeOk = A.tcPlan && B.tcPlan && A.convK == 1 && B.convK == 1 && A.convInStride == A.convInC &&
                           B.convIn == ea.outAct && B.convInStride == A.convOutC && B.convInC == A.convOutC;
      const bool aOk = shapeOk && ea.residual && ea.residual == ea.outRaw && ea.resStride == A.convOutC && !ea.resMask && !ea.biasNC &&
                       ea.rawC0 == 0 && ea.rawC1 == A.convOutC && ea.rawStride == A.convOutC && ea.outAct && ea.actC0 == 0 &&
                       ea.actC1 == A.convOutC && ea.actStride == A.convOutC && !ea.sumsqOut && !ea.rowSumsq && ea.act != KB_ACT_SWIGLU_PAIRS;
      const bool bOk = aOk && !eb.residual && !eb.biasNC && eb.outRaw && eb.outAct && eb.rawC0 == 0 && eb.rawC1 == B.convOutC &&
                       eb.rawStride == B.convOutC && eb.actC0 == 0 && eb.actC1 == B.convOutC && eb.actStride == B.convOutC &&
                       !eb.sumsqOut && !eb.rowSumsq && eb.act == ea.act;
      if(bOk && convPostPreEligible(dt_, A.convInC, A.convOutC, B.convOutC)) {
        plan = convPostPreCreate(dt_, A.convIn, A.convInC, A.convW, ea.outRaw, A.convOutC, ea.scale, ea.bias, ea.act, B.convW, eb.outRaw,
                                 eb.outAct, B.convOutC, eb.scale, eb.bias, eb.act, mask_, rowsPadMax_);
      }
    }
    if(plan) {
      postPrePlans_.push_back(plan);
      Op op;
      op.flops = ops_[i].flops + ops_[i + 1].flops;
      const double S = (double)X_ * Y_, es = (double)dtypeSize(dt_);
      op.bytes = S * es * (ops_[i].convInC + 2.0 * ops_[i].convOutC + 2.0 * ops_[i + 1].convOutC);
      op.cls = classId("conv1x1 " + std::to_string(ops_[i].convInC) + "->" + std::to_string(ops_[i].convOutC) + " +res | 1x1 ->" +
                       std::to_string(ops_[i + 1].convOutC) + " tcgen05 fused");
      int* status = statusWord_;
      op.run = [plan, status](cudaStream_t st, const Geom& g) { return launchConvPostPre(st, plan, g, status); };
      out.push_back(std::move(op));
      i += 2;
    }
    else {
      out.push_back(ops_[i]);
      i++;
    }
  }
  if(!postPrePlans_.empty()) ops_ = std::move(out);
}

// Replaces every run of two or more consecutive chainable tensor-core convolutions of the launch list by one
// multi-layer launch (kb_conv_tc.cu, convChainKernel).  Between two members of a run nothing else is launched, so the
// only producers of a member's inputs inside the run are the members before it, and their hand-over is per tile.
void Engine::planChains() {
  chainMode_ = getenv("KB_CHAIN") != nullptr ? atoi(getenv("KB_CHAIN")) : 1;
  if(chainMode_ <= 0 || chunkBoards_ > 0 || layerN_ != 0 || forceSimt_) return;
  const size_t tiles = (size_t)rowsPadMax_ / 128;
  auto chainable = [&](const Op& op) {
    return op.tcPlan && convChainEligible(op.tcPlan, op.ep) && (chainMode_ >= 2 || convTcChainPreferred(op.tcPlan));
  };
  // counters: one array per chain member
  size_t members = 0;
  for(const Op& op : ops_) if(chainable(op)) members++;
  if(members < 2) return;
  tileCtrBytes_ = members * tiles * sizeof(uint32_t);
  tileCtr_ = static_cast<uint32_t*>(alloc(tileCtrBytes_));
  size_t ctrIdx = 0;
  std::vector<Op> out;
  size_t i = 0;
  while(i < ops_.size()) {
    size_t j = i;
    while(j < ops_.size() && chainable(ops_[j]) && j - i < 16 &&
          (j == i || (convTcTileWidth(ops_[j].tcPlan) == convTcTileWidth(ops_[i].tcPlan) &&
                      (!ops_[j].ep.outAct || !ops_[i].ep.outAct || ops_[j].ep.act == ops_[i].ep.act))))
      j++;
    ConvChainPlan* plan = nullptr;
    if(j - i >= 2) {
      std::vector<ConvChainMember> ms;
      for(size_t k = i; k < j; k++) {
        ConvChainMember m;
        m.plan = ops_[k].tcPlan;
        m.ep = ops_[k].ep;
        m.done = tileCtr_ + (ctrIdx++) * tiles;
        ms.push_back(m);
      }
      plan = convChainCreate(ms.data(), (int)ms.size());
    }
    if(plan) {
      chainPlans_.push_back(plan);
      Op op;
      size_t big = i;
      for(size_t k = i; k < j; k++) {
        op.flops += ops_[k].flops;
        op.bytes += ops_[k].bytes;
        if(ops_[k].flops > ops_[big].flops) big = k;
      }
      op.cls = classId(classes_[ops_[big].cls].name + " chain x" + std::to_string(j - i));
      int* status = statusWord_;
      op.run = [plan, status](cudaStream_t st, const Geom& g) { return launchConvChain(st, plan, g, status); };
      out.push_back(std::move(op));
      i = j;
    }
    else {
      out.push_back(ops_[i]);
      i++;
    }
  }
  if(chainPlans_.empty()) return;
  ops_ = std::move(out);
}

void Engine::planTileDeps() {
  if(!tileDeps_ || chunkBoards_ > 0 || layerN_ != 0) return;
  const size_t tiles = (size_t)rowsPadMax_ / 128;
  size_t numTc = 0;
  auto reports = [&](const Op& op) {
    return op.tcPlan && convTcDepsCapable(op.tcPlan) && (tileDepsMode_ >= 2 || convTcKernelSize(op.tcPlan) == 3);
  };
  for(const Op& op : ops_) if(reports(op)) numTc++;
  if(numTc == 0) return;
  tileCtrBytes_ = numTc * tiles * sizeof(uint32_t);
  tileCtr_ = static_cast<uint32_t*>(alloc(tileCtrBytes_));
  size_t idx = 0;
  for(Op& op : ops_)
    if(reports(op)) op.deps->done = tileCtr_ + (idx++) * tiles;
  for(size_t i = 1; i < ops_.size(); i++) {
    Op& cur = ops_[i];
    const Op& prev = ops_[i - 1];
    if(!cur.tcPlan || !prev.tcPlan || !convTcDepsCapable(cur.tcPlan) || !prev.deps->done) continue;
    const Epilogue& e = cur.ep;
    if(e.biasNC || e.rowSumsq || e.sumsqOut || prev.ep.sumsqOut || prev.ep.rowSumsq) continue;
    if(e.act == KB_ACT_SWIGLU_PAIRS || prev.ep.act == KB_ACT_SWIGLU_PAIRS) continue;  // no such kernel variant
    if(e.act == KB_ACT_ROPE_QK || prev.ep.act == KB_ACT_ROPE_QK) continue;
    if(e.residual) {
      const int r = allocationOf(e.residual);
      if(r < 0 || r == allocationOf(prev.ep.outRaw) || r == allocationOf(prev.ep.outAct)) continue;
    }
    cur.deps->wait = prev.deps->done;
    cur.deps->waitPlan = prev.tcPlan;
  }
}

void Engine::selfTestWaitTimeout(unsigned long long limitNs) {
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  cudaCheck(launchWaitTimeoutSelfTest(stream_, statusWord_, limitNs), "wait self-test launch");
  cudaCheck(cudaMemcpyAsync(statusHost_, statusWord_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "status copy");
  sync();
}

void Engine::launchOpsEager(int n) {
  // Optionally (KB_CHUNK_BOARDS) the batch runs through the launch list in chunks of boards that reuse the same
  // activation buffers, so that tensors handed from kernel to kernel stay in the 126 MB L2.
  const int chunk = (chunkBoards_ > 0 && layerN_ == 0) ? chunkBoards_ : n;
  for(int c0 = 0; c0 < n; c0 += chunk) {
    const int nc = std::min(chunk, n - c0);
    boardOffset_ = c0;
    const Geom g = makeGeom(X_, Y_, nc);
    if(tileCtr_) cudaCheck(cudaMemsetAsync(tileCtr_, 0, tileCtrBytes_, stream_), "reset of the tile counters");
    for(size_t i = 0; i < ops_.size(); i++) {
      if(profiling_) cudaCheck(cudaEventRecord(events_[2 * i], stream_), "event record");
      cudaError_t e = ops_[i].run(stream_, g);
      if(e != cudaSuccess) throw CudaError("launch of '" + classes_[ops_[i].cls].name + "' failed: " + cudaGetErrorString(e));
      if(profiling_) cudaCheck(cudaEventRecord(events_[2 * i + 1], stream_), "event record");
    }
    if(profiling_) {
      cudaCheck(cudaStreamSynchronize(stream_), "stream synchronize");
      for(size_t i = 0; i < ops_.size(); i++) {
        float ms = 0.0f;
        cudaCheck(cudaEventElapsedTime(&ms, events_[2 * i], events_[2 * i + 1]), "event elapsed");
        OpClass& c = classes_[ops_[i].cls];
        c.launches += 1;
        c.ms += ms;
        c.flops += ops_[i].flops * nc;
        c.bytes += ops_[i].bytes * nc;
      }
    }
  }
  boardOffset_ = 0;
}

void Engine::runOps(int n) {
  if(n < 1 || n > maxBatch_) throw std::runtime_error("batch size out of range for this handle");
  if(profiling_ && events_.size() < 2 * ops_.size()) {
    size_t old = events_.size();
    events_.resize(2 * ops_.size());
    for(size_t i = old; i < events_.size(); i++) cudaCheck(cudaEventCreate(&events_[i]), "cudaEventCreate");
  }
  // Whole-network runs replay a CUDA graph of the launch list from the second run of a batch size on: the kernels'
  // arguments depend only on the batch size and on whether symmetries were uploaded.
  const bool graphable = graphsEnabled_ && !profiling_ && layerN_ == 0 && chunkBoards_ == 0;
  bool done = false;
  if(graphable) {
    GraphEntry& ge = graphs_[n * 2 + (haveSym_ ? 1 : 0)];
    if(ge.exec) {
      cudaCheck(cudaGraphLaunch(ge.exec, stream_), "cudaGraphLaunch");
      done = true;
    }
    else if(++ge.uses >= 2 && graphsInstantiated_ < 64) {
      cudaGraph_t graph = nullptr;
      bool ok = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      if(ok) {
        try { launchOpsEager(n); }
        catch(...) { ok = false; }
        if(cudaStreamEndCapture(stream_, &graph) != cudaSuccess) ok = false;
      }
      if(ok && graph && cudaGraphInstantiate(&ge.exec, graph, 0) == cudaSuccess) {
        graphsInstantiated_++;
        cudaCheck(cudaGraphLaunch(ge.exec, stream_), "cudaGraphLaunch");
        done = true;
      }
      else {
        // capture is not possible here: stay eager for good
        ge.exec = nullptr;
        graphsEnabled_ = false;
        cudaGetLastError();
      }
      if(graph) cudaGraphDestroy(graph);
    }
  }
  if(!done) launchOpsEager(n);
  cudaCheck(cudaMemcpyAsync(statusHost_, statusWord_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "status copy");
  if(profiling_) sync();
}

void Engine::uploadInputs(int n, const float* spatial, const float* global, const int32_t* symmetry, const float* meta) {
  if(n < 1 || n > maxBatch_) throw std::runtime_error("batch size out of range for this handle");
  if(!spatial || !global) throw std::runtime_error("NULL input pointer");
  if(inMetaC_ > 0 && !meta) throw std::runtime_error("this model has an SGF metadata encoder: metadata input rows are required");
  if(inMetaC_ == 0 && meta) throw std::runtime_error("this model has no SGF metadata encoder: metadata input rows must be NULL");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  const size_t S = (size_t)X_ * Y_;
  cudaCheck(cudaMemcpyAsync(dSpatial_, spatial, (size_t)n * S * inC_ * sizeof(float), cudaMemcpyHostToDevice, stream_), "H2D spatial");
  cudaCheck(cudaMemcpyAsync(dGlobal_, global, (size_t)n * inGlobalC_ * sizeof(float), cudaMemcpyHostToDevice, stream_), "H2D global");
  if(meta) cudaCheck(cudaMemcpyAsync(dMeta_, meta, (size_t)n * inMetaC_ * sizeof(float), cudaMemcpyHostToDevice, stream_), "H2D metadata");
  haveSym_ = symmetry != nullptr;
  if(symmetry) {
    for(int i = 0; i < n; i++)
      if(symmetry[i] < 0 || symmetry[i] > 7) throw std::runtime_error("symmetry index out of range");
    cudaCheck(cudaMemcpyAsync(dSym_, symmetry, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, stream_), "H2D symmetry");
  }
}

void Engine::forwardResident(int n) {
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  runOps(n);
}

void Engine::downloadOutputs(int n, float* policy, float* policyPass, float* value, float* scoreValue, float* ownership) {
  if(n < 1 || n > maxBatch_) throw std::runtime_error("batch size out of range for this handle");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  const size_t S = (size_t)X_ * Y_;
  if(policy) cudaCheck(cudaMemcpyAsync(policy, dPolicy_, (size_t)n * S * policyC_ * 4, cudaMemcpyDeviceToHost, stream_), "D2H policy");
  if(policyPass) cudaCheck(cudaMemcpyAsync(policyPass, dPolicyPass_, (size_t)n * policyC_ * 4, cudaMemcpyDeviceToHost, stream_), "D2H pass");
  if(value) cudaCheck(cudaMemcpyAsync(value, dValue_, (size_t)n * valueC_ * 4, cudaMemcpyDeviceToHost, stream_), "D2H value");
  if(scoreValue) cudaCheck(cudaMemcpyAsync(scoreValue, dScore_, (size_t)n * scoreValueC_ * 4, cudaMemcpyDeviceToHost, stream_), "D2H score");
  if(ownership) cudaCheck(cudaMemcpyAsync(ownership, dOwnership_, (size_t)n * S * 4, cudaMemcpyDeviceToHost, stream_), "D2H ownership");
  sync();
}

float Engine::timeForwardResident(int n, int iters) {
  if(iters < 1) throw std::runtime_error("iters must be positive");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  cudaEvent_t a, b;
  cudaCheck(cudaEventCreate(&a), "cudaEventCreate");
  cudaCheck(cudaEventCreate(&b), "cudaEventCreate");
  const bool wasProfiling = profiling_;
  profiling_ = false;
  cudaCheck(cudaEventRecord(a, stream_), "event record");
  for(int i = 0; i < iters; i++) runOps(n);
  cudaCheck(cudaEventRecord(b, stream_), "event record");
  profiling_ = wasProfiling;
  sync();
  float ms = 0.0f;
  cudaCheck(cudaEventElapsedTime(&ms, a, b), "event elapsed");
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return ms / iters;
}

void Engine::timeForwardSteps(int n, int steps, size_t flushBytes, float* msEach) {
  if(steps < 1 || steps > 100000) throw std::runtime_error("steps out of range");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  if(flushBytes > flushBytes_) {
    if(flushBuf_) cudaFree(flushBuf_);
    flushBuf_ = nullptr;
    flushBytes_ = 0;
    cudaCheck(cudaMalloc(&flushBuf_, flushBytes), "cudaMalloc flush buffer");
    flushBytes_ = flushBytes;
  }
  std::vector<cudaEvent_t> ev(2 * (size_t)steps);
  for(auto& e : ev) cudaCheck(cudaEventCreate(&e), "cudaEventCreate");
  const bool wasProfiling = profiling_;
  profiling_ = false;
  for(int i = 0; i < steps; i++) {
    if(flushBytes > 0) cudaCheck(cudaMemsetAsync(flushBuf_, i & 0xff, flushBytes, stream_), "L2 flush");
    cudaCheck(cudaEventRecord(ev[2 * i], stream_), "event record");
    runOps(n);
    cudaCheck(cudaEventRecord(ev[2 * i + 1], stream_), "event record");
  }
  profiling_ = wasProfiling;
  sync();
  for(int i = 0; i < steps; i++) cudaCheck(cudaEventElapsedTime(&msEach[i], ev[2 * i], ev[2 * i + 1]), "event elapsed");
  for(auto& e : ev) cudaEventDestroy(e);
}

void Engine::readTrunk(int n, float* out) {
  if(!trunkAct_ || !out) throw std::runtime_error("no trunk buffer");
  if(chunkBoards_ > 0 && n > chunkBoards_) throw std::runtime_error("the trunk buffer only holds the last chunk of boards; read it with n <= the chunk size");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  const Geom g = makeGeom(X_, Y_, n);
  float* tmp = nullptr;
  const size_t bytes = (size_t)n * g.S * trunkC_ * sizeof(float);
  cudaCheck(cudaMalloc(&tmp, bytes), "cudaMalloc");
  cudaError_t e = launchFromPadded(stream_, dt_, trunkAct_, trunkC_, trunkC_, tmp, g);
  if(e == cudaSuccess) e = cudaMemcpyAsync(out, tmp, bytes, cudaMemcpyDeviceToHost, stream_);
  if(e == cudaSuccess) e = cudaStreamSynchronize(stream_);
  cudaFree(tmp);
  cudaCheck(e, "read trunk");
}

void Engine::profileReset() {
  for(OpClass& c : classes_) { c.launches = 0; c.ms = 0.0; c.flops = 0.0; c.bytes = 0.0; }
}

int Engine::profileRead(OpClass* out, int cap) {
  int k = 0;
  for(const OpClass& c : classes_) {
    if(k >= cap) break;
    out[k++] = c;
  }
  return k;
}

// ---------------------------------------------------------------------------------------------
// Single-layer mode

Engine::Engine(const void* layerBlob, size_t nbytes, int device, int n, int X, int Y, int precision) {
  if(n < 1 || n > 65536) throw std::runtime_error("batch size out of range");
  if(X < 1 || Y < 1 || X > 50 || Y > 50) throw std::runtime_error("board size out of range");
  if(precision != DT_F32 && precision != DT_F16 && precision != DT_BF16) throw std::runtime_error("unknown precision");
  device_ = pickDevice(device);
  dt_ = precision; X_ = X; Y_ = Y; maxBatch_ = n; layerN_ = n;
  forceSimt_ = getenv("KB_FORCE_SIMT") != nullptr && atoi(getenv("KB_FORCE_SIMT")) != 0;
  cudaCheck(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  const Geom g = makeGeom(X, Y, n);
  rowsPadMax_ = g.rowsPad;
  const size_t es = dtypeSize(dt_);
  const size_t S = (size_t)X * Y;
  statusWord_ = static_cast<int*>(alloc(sizeof(int)));
  cudaCheck(cudaHostAlloc(reinterpret_cast<void**>(&statusHost_), sizeof(int), cudaHostAllocDefault), "cudaHostAlloc");
  *statusHost_ = 0;
  mask_ = static_cast<float*>(alloc((size_t)rowsPadMax_ * sizeof(float)));
  maskSum_ = static_cast<float*>(alloc((size_t)n * sizeof(float)));
  layerMaskIn_ = static_cast<float*>(alloc((size_t)n * S * sizeof(float)));

  kbblob::Reader rd(layerBlob, nbytes);
  const uint32_t tag = rd.peekTag();
  const int dt = dt_;
  if(tag == KB_TAG_CONV) {
    ConvW cw;
    parseConv(rd, cw);
    layerInC_ = cw.inC; layerOutC_ = cw.outC;
    // pad the channel stride so that the tensor-core path is exercised when the shape allows it
    const bool tcOk = !forceSimt_ && dt_ != DT_F32 && convTcEligible(dt_, (cw.inC + 63) / 64 * 64, cw.outC, cw.kY, cw.kX);
    const int inCdev = tcOk ? (cw.inC + 63) / 64 * 64 : cw.inC;
    void* inBuf = alloc((size_t)rowsPadMax_ * inCdev * es);
    void* outBuf = alloc((size_t)rowsPadMax_ * cw.outC * es);
    layerIn_ = static_cast<float*>(alloc((size_t)n * S * cw.inC * sizeof(float)));
    layerOut_ = static_cast<float*>(alloc((size_t)n * S * cw.outC * sizeof(float)));
    const int inC = cw.inC, outC = cw.outC;
    float* lin = layerIn_; float* lout = layerOut_;
    addOp("to padded", 0, 0, [=](cudaStream_t st, const Geom& gg) { return launchToPadded(st, dt, lin, inC, inBuf, inCdev, gg); });
    ConvDev c = makeConv({&cw}, inBuf, inCdev, inCdev);
    Epilogue e;
    e.outRaw = outBuf; e.rawStride = outC; e.rawC0 = 0; e.rawC1 = outC;
    addConvOp(c, e, "layer");
    addOp("from padded", 0, 0, [=](cudaStream_t st, const Geom& gg) { return launchFromPadded(st, dt, outBuf, outC, outC, lout, gg); });
    // a bare convolution has no mask: the epilogue must not read one
    layerNeedsMask_ = false;
  }
  else if(tag == KB_TAG_BN) {
    BNW bw;
    parseBN(rd, bw);
    layerInC_ = bw.C; layerOutC_ = bw.C;
    const int C = bw.C;
    void* inBuf = alloc((size_t)rowsPadMax_ * C * es);
    void* outBuf = alloc((size_t)rowsPadMax_ * C * es);
    layerIn_ = static_cast<float*>(alloc((size_t)n * S * C * sizeof(float)));
    layerOut_ = static_cast<float*>(alloc((size_t)n * S * C * sizeof(float)));
    BNDev b = makeBN({&bw});
    float* lin = layerIn_; float* lout = layerOut_; float* mask = mask_;
    addOp("to padded", 0, 0, [=](cudaStream_t st, const Geom& gg) { return launchToPadded(st, dt, lin, C, inBuf, C, gg); });
    addOp("norm+act", 0, 0, [=](cudaStream_t st, const Geom& gg) {
      return launchBnAct(st, dt, inBuf, C, b.scale, b.bias, b.act, mask, dt, outBuf, C, C, gg);
    });
    addOp("from padded", 0, 0, [=](cudaStream_t st, const Geom& gg) { return launchFromPadded(st, dt, outBuf, C, C, lout, gg); });
    layerNeedsMask_ = true;
  }
  else {
    BlockW bw;
    parseBlock(rd, bw);
    const int C = bw.channels();
    layerInC_ = C; layerOutC_ = C;
    void* raw = alloc((size_t)rowsPadMax_ * C * es);
    void* act = alloc((size_t)rowsPadMax_ * C * es);
    layerIn_ = static_cast<float*>(alloc((size_t)n * S * C * sizeof(float)));
    layerOut_ = static_cast<float*>(alloc((size_t)n * S * C * sizeof(float)));
    BNDev pb;
    if(isConvBlock(bw)) pb = makeBN({&bw.preBN});
    float* lin = layerIn_; float* lout = layerOut_; float* mask = mask_;
    addOp("to padded", 0, 0, [=](cudaStream_t st, const Geom& gg) { return launchToPadded(st, dt, lin, C, raw, C, gg); });
    if(isConvBlock(bw)) {
      addOp("norm+act", 0, 0, [=](cudaStream_t st, const Geom& gg) {
        return launchBnAct(st, dt, raw, C, pb.scale, pb.bias, pb.act, mask, dt, act, C, C, gg);
      });
    }
    emitBlock(bw, C, raw, act, nullptr, 0);
    addOp("from padded", 0, 0, [=](cudaStream_t st, const Geom& gg) { return launchFromPadded(st, dt, raw, C, C, lout, gg); });
    layerNeedsMask_ = true;
  }
  cudaCheck(cudaStreamSynchronize(stream_), "engine setup");
}

void Engine::evalLayer(const float* in, const float* mask, float* out) {
  if(!in || !out) throw std::runtime_error("NULL pointer");
  if(layerNeedsMask_ && !mask) throw std::runtime_error("this layer needs a mask");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  const Geom g = makeGeom(X_, Y_, layerN_);
  const size_t S = (size_t)X_ * Y_;
  cudaCheck(cudaMemcpyAsync(layerIn_, in, (size_t)layerN_ * S * layerInC_ * 4, cudaMemcpyHostToDevice, stream_), "H2D layer input");
  if(mask) {
    cudaCheck(cudaMemcpyAsync(layerMaskIn_, mask, (size_t)layerN_ * S * 4, cudaMemcpyHostToDevice, stream_), "H2D layer mask");
    cudaCheck(launchMaskToPadded(stream_, layerMaskIn_, mask_, maskSum_, g), "mask to padded");
  }
  else {
    // all-ones mask on board points (padding rows stay 0)
    std::vector<float> ones((size_t)layerN_ * S, 1.0f);
    cudaCheck(cudaMemcpyAsync(layerMaskIn_, ones.data(), ones.size() * 4, cudaMemcpyHostToDevice, stream_), "H2D ones");
    cudaCheck(cudaStreamSynchronize(stream_), "sync");
    cudaCheck(launchMaskToPadded(stream_, layerMaskIn_, mask_, maskSum_, g), "mask to padded");
  }
  runOps(layerN_);
  cudaCheck(cudaMemcpyAsync(out, layerOut_, (size_t)layerN_ * S * layerOutC_ * 4, cudaMemcpyDeviceToHost, stream_), "D2H layer output");
  sync();
}

}  // namespace kb
