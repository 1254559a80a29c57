// kb_conv_noalloc: a convolution entry point that never allocates.
//
// Who needs it: code that runs inside somebody else's memory regime -- a host framework that hands out
// device buffers from its own pool and forbids cudaMalloc on its threads, or a real-time loop that must not
// take the allocator's locks or trigger the implicit device synchronisation a cudaMalloc/cudaFree can cause.
// Such a caller already owns device buffers for the input, the weights and the output, but the convolution
// also needs working memory (the padded-row copies of input and output and the re-ordered weights).  Here
// that working memory is a fixed array in the library's own device image, so nothing is requested at run
// time.  The price is a hard size limit and the fact that the array is shared by every call.
#include "../../include/katab200.h"
#include "kb_kernels.cuh"

#include <mutex>
#include <string>

namespace {

constexpr int NA_MAX_ROWS = 4096;      // padded rows: n*(Y+1)*(X+1) rounded up to 256
constexpr int NA_MAX_CHANNELS = 64;    // input and output channels
constexpr int NA_MAX_TAPS = 25;        // up to 5x5
constexpr size_t NA_IN_FLOATS = (size_t)NA_MAX_ROWS * NA_MAX_CHANNELS;
constexpr size_t NA_OUT_FLOATS = (size_t)NA_MAX_ROWS * NA_MAX_CHANNELS;
constexpr size_t NA_W_FLOATS = (size_t)NA_MAX_TAPS * NA_MAX_CHANNELS * NA_MAX_CHANNELS;

// The working memory: 2.4 MiB held by every GPU that loads the library, until the process exits.
// In host code this name is only a stand-in for the device object; the usable device address comes from
// cudaGetSymbolAddress (deviceScratch below).
static __device__ __align__(256) float g_noallocScratch[NA_IN_FLOATS + NA_OUT_FLOATS + NA_W_FLOATS];

constexpr int NA_MAX_DEVICES = 64;
std::mutex g_naMutex;
float* g_naAddr[NA_MAX_DEVICES] = {nullptr};

thread_local std::string g_naErr;

// weights [oc][ic][y][x] (the reference's ConvLayerDesc order) -> [tap][ic][oc], the order the CUDA-core kernel reads
__global__ void repackWeightsKernel(const float* __restrict__ src, float* __restrict__ dst, int inC, int outC, int taps) {
  const int total = taps * inC * outC;
  for(int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int oc = i % outC, ic = (i / outC) % inC, tap = i / (outC * inC);
    dst[i] = src[((size_t)oc * inC + ic) * taps + tap];
  }
}

// Device address of the scratch array on the current device; resolved once per device.
cudaError_t deviceScratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if(e != cudaSuccess) return e;
  if(dev < 0 || dev >= NA_MAX_DEVICES) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_naMutex);
  if(g_naAddr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noallocScratch);
    if(e != cudaSuccess) return e;
    g_naAddr[dev] = p;
  }
  *out = g_naAddr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" {

const char* kb_conv_noalloc_last_error(void) { return g_naErr.c_str(); }

int kb_conv_noalloc(
  const float* dIn, const float* dWeights, float* dOut, int n, int nnXLen, int nnYLen, int inC, int outC, int kY, int kX,
  void* stream) {
  if(!dIn || !dWeights || !dOut) { g_naErr = "kb_conv_noalloc: NULL device pointer"; return 1; }
  if(n < 1 || nnXLen < 1 || nnYLen < 1 || nnXLen > 50 || nnYLen > 50) { g_naErr = "kb_conv_noalloc: bad batch or board size"; return 1; }
  if(kY < 1 || kX < 1 || (kY % 2) != 1 || (kX % 2) != 1 || kY * kX > NA_MAX_TAPS) {
    g_naErr = "kb_conv_noalloc: kernel size must be odd and at most 5x5";
    return 1;
  }
  if(inC < 1 || outC < 1 || inC > NA_MAX_CHANNELS || outC > NA_MAX_CHANNELS) {
    g_naErr = "kb_conv_noalloc: at most " + std::to_string(NA_MAX_CHANNELS) + " input and output channels fit the built-in scratch";
    return 1;
  }
  const kb::Geom g = kb::makeGeom(nnXLen, nnYLen, n);
  if(g.rowsPad > NA_MAX_ROWS) {
    g_naErr = "kb_conv_noalloc: n*(Y+1)*(X+1) = " + std::to_string(g.rows) + " padded rows exceed the built-in scratch of " +
              std::to_string(NA_MAX_ROWS) + " rows";
    return 1;
  }
  float* scratch = nullptr;
  cudaError_t e = deviceScratch(&scratch);
  if(e != cudaSuccess) { g_naErr = std::string("kb_conv_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e); return 2; }
  float* sIn = scratch;
  float* sOut = scratch + NA_IN_FLOATS;
  float* sW = scratch + NA_IN_FLOATS + NA_OUT_FLOATS;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int taps = kY * kX;
  // Nothing in the scratch has to start at zero: the padded copy is written for every board point before it is
  // read, the convolution reads board points only (padding is handled by coordinates), and the output copy is
  // fully overwritten.  Whatever the previous call left behind is never read.
  e = kb::launchToPadded(st, kb::DT_F32, dIn, inC, sIn, inC, g);
  if(e == cudaSuccess) {
    const int total = taps * inC * outC;
    repackWeightsKernel<<<(total + 255) / 256, 256, 0, st>>>(dWeights, sW, inC, outC, taps);
    e = cudaGetLastError();
  }
  if(e == cudaSuccess) {
    kb::Epilogue ep;
    ep.outRaw = sOut; ep.rawStride = outC; ep.rawC0 = 0; ep.rawC1 = outC;
    e = kb::launchConvSimt(st, kb::DT_F32, sIn, inC, inC, sW, outC, kY, kX, g, ep);
  }
  if(e == cudaSuccess) e = kb::launchFromPadded(st, kb::DT_F32, sOut, outC, outC, dOut, g);
  if(e != cudaSuccess) { g_naErr = std::string("kb_conv_noalloc: launch failed: ") + cudaGetErrorString(e); return 2; }
  return 0;
}

}  // extern "C"
