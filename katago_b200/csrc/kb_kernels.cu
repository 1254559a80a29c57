// CUDA-core kernels: input packing, the generic convolution used for fp32 and for shapes the
// tensor-core kernel does not take, masked global pooling, the fused bias+norm+activation pass of
// the gpool blocks, the small per-board matmuls and the head outputs.  All are bandwidth-bound
// except the convolution; rows are channel-contiguous (NHWC), so adjacent threads read adjacent
// channels.
#include "kb_kernels.cuh"
#include "kb_act.cuh"
#include "../../include/kb_modelblob.h"

namespace kb {

// ---------------------------------------------------------------------------------------------
// dtype helpers

template <typename T> __device__ __forceinline__ float toF(T v);
template <> __device__ __forceinline__ float toF<float>(float v) { return v; }
template <> __device__ __forceinline__ float toF<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float toF<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T fromF(float v);
template <> __device__ __forceinline__ float fromF<float>(float v) { return v; }
template <> __device__ __forceinline__ __half fromF<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 fromF<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Activation functions (eigenbackend.cpp:749-760; MISH_SCALE8 from desc.cpp:402-432).
__device__ __forceinline__ float mishF(float x) {
  // x * tanh(softplus(x)), softplus linear above 20
  float sp = (x > 20.0f) ? x : log1pf(expf(x));
  return x * tanhf(sp);
}
__device__ __forceinline__ float applyActF(float x, int act) {
  switch(act) {
    case KB_ACT_RELU: return fmaxf(x, 0.0f);
    case KB_ACT_MISH: return mishF(x);
    case KB_ACT_SILU: return x / (1.0f + expf(-x));
    case KB_ACT_MISH_SCALE8: {
      float x8 = 8.0f * x;
      float sp = (x8 > 20.0f) ? x8 : log1pf(expf(x8));
      return x * tanhf(sp);
    }
    default: return x;
  }
}

// Board symmetry as a point map (h,w) -> (h',w'), the scatter form of nninputs.cpp:529-575.
// `reverse` = false for inputs, true for outputs (the flips swap roles under transposition only for inputs).
__device__ __forceinline__ void symMap(int sym, bool reverse, int H, int W, int h, int w, int& h2, int& w2) {
  bool transpose = (sym & 4) != 0 && H == W;
  bool flipX = (sym & 2) != 0;
  bool flipY = (sym & 1) != 0;
  if(transpose && !reverse) { bool t = flipX; flipX = flipY; flipY = t; }
  if(!transpose) {
    h2 = flipY ? H - 1 - h : h;
    w2 = flipX ? W - 1 - w : w;
  }
  else {
    h2 = flipY ? H - 1 - w : w;
    w2 = flipX ? W - 1 - h : h;
  }
}

#define KB_DISPATCH_DT(dt, EXPR)                                   \
  switch(dt) {                                                     \
    case DT_F32: { using T = float; EXPR; break; }                 \
    case DT_F16: { using T = __half; EXPR; break; }                \
    case DT_BF16: { using T = __nv_bfloat16; EXPR; break; }        \
    default: return cudaErrorInvalidValue;                         \
  }

// ---------------------------------------------------------------------------------------------
// Input packing

template <typename T>
__global__ void packInputKernel(
  const float* __restrict__ spatial, const int32_t* __restrict__ symmetry, int inC, T* __restrict__ dst, int dstStride,
  float* __restrict__ mask, float* __restrict__ maskSum, Geom g) {
  const int n = blockIdx.x;
  const int sym = symmetry ? symmetry[n] : 0;
  float localSum = 0.0f;
  const float* src = spatial + (size_t)n * g.S * inC;
  // one thread per (point, channel); channel fastest so reads are contiguous
  for(int idx = threadIdx.x; idx < g.S * inC; idx += blockDim.x) {
    int p = idx / inC, c = idx - p * inC;
    int h = p / g.X, w = p - h * g.X;
    int h2, w2;
    symMap(sym, false, g.Y, g.X, h, w, h2, w2);
    size_t row = (size_t)n * g.PB + (size_t)h2 * g.RW + w2;
    float v = src[idx];
    dst[row * dstStride + c] = fromF<T>(v);
    if(c == 0) { mask[row] = v; localSum += v; }
  }
  // padding rows of the mask stay 0 from allocation time; block-reduce the mask sum
  __shared__ float red[32];
  for(int o = 16; o > 0; o >>= 1) localSum += __shfl_down_sync(0xffffffffu, localSum, o);
  if((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = localSum;
  __syncthreads();
  if(threadIdx.x < 32) {
    float v = (threadIdx.x < (blockDim.x + 31) / 32) ? red[threadIdx.x] : 0.0f;
    for(int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if(threadIdx.x == 0) maskSum[n] = v;
  }
}

// Reduced-precision variant for inC <= 32 and rows of at least 32 channels: one thread per board point reads its inC
// floats and writes 32 channels (64 bytes) with four 16-byte stores; the rest of the row stays zero from allocation.
template <typename T>
__global__ void __launch_bounds__(384) packInputVecKernel(
  const float* __restrict__ spatial, const int32_t* __restrict__ symmetry, int inC, T* __restrict__ dst, int dstStride,
  float* __restrict__ mask, float* __restrict__ maskSum, Geom g) {
  const int n = blockIdx.x;
  const int sym = symmetry ? symmetry[n] : 0;
  const float* src = spatial + (size_t)n * g.S * inC;
  float localSum = 0.0f;
  for(int p = threadIdx.x; p < g.S; p += blockDim.x) {
    const int h = p / g.X, w = p - h * g.X;
    int h2, w2;
    symMap(sym, false, g.Y, g.X, h, w, h2, w2);
    const size_t row = (size_t)n * g.PB + (size_t)h2 * g.RW + w2;
    float v[32];
#pragma unroll
    for(int c = 0; c < 32; c++) v[c] = c < inC ? src[(size_t)p * inC + c] : 0.0f;
    uint4 o[4];
    T* oe = reinterpret_cast<T*>(o);
#pragma unroll
    for(int c = 0; c < 32; c++) oe[c] = fromF<T>(v[c]);
    uint4* d = reinterpret_cast<uint4*>(dst + row * dstStride);
#pragma unroll
    for(int k = 0; k < 4; k++) d[k] = o[k];
    mask[row] = v[0];
    localSum += v[0];
  }
  __shared__ float red[32];
  for(int o = 16; o > 0; o >>= 1) localSum += __shfl_down_sync(0xffffffffu, localSum, o);
  if((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = localSum;
  __syncthreads();
  if(threadIdx.x < 32) {
    float v = (threadIdx.x < (blockDim.x + 31) / 32) ? red[threadIdx.x] : 0.0f;
    for(int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if(threadIdx.x == 0) maskSum[n] = v;
  }
}

cudaError_t launchPackInput(
  cudaStream_t st, int dt, const float* spatial, const int32_t* symmetry, int inC, void* dst, int dstStride,
  float* mask, float* maskSum, Geom g) {
  if(dt != DT_F32 && inC <= 32 && dstStride >= 32 && (dstStride % 8) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    if(dt == DT_F16) packInputVecKernel<__half><<<g.n, 384, 0, st>>>(spatial, symmetry, inC, (__half*)dst, dstStride, mask, maskSum, g);
    else packInputVecKernel<__nv_bfloat16><<<g.n, 384, 0, st>>>(spatial, symmetry, inC, (__nv_bfloat16*)dst, dstStride, mask, maskSum, g);
    return cudaGetLastError();
  }
  KB_DISPATCH_DT(dt, (packInputKernel<T><<<g.n, 256, 0, st>>>(spatial, symmetry, inC, (T*)dst, dstStride, mask, maskSum, g)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Generic convolution (CUDA cores).  Block tile 64 rows x 64 output channels, 256 threads, each
// thread 4 rows x 4 channels; K loop over taps and chunks of 16 input channels staged in shared memory.

constexpr int SC_BM = 64, SC_BN = 64, SC_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256) convSimtKernel(
  const T* __restrict__ in, int inStride, int inC, const T* __restrict__ w, int outC, int kY, int kX, Geom g, Epilogue ep) {
  __shared__ float sA[SC_BK][SC_BM + 4];
  __shared__ float sB[SC_BK][SC_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * SC_BM, n0 = blockIdx.y * SC_BN;
  const int padY = kY / 2, padX = kX / 2;

  // The A-tile element this thread stages: row lr (0..63), 4 consecutive k's starting at lk.
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int lm = m0 + lr;
  const int lb = lm / g.PB, lrem = lm - lb * g.PB;
  const int ly = lrem / g.RW, lx = lrem - ly * g.RW;
  const bool lvalid = lm < g.rows && ly < g.Y && lx < g.X;
  // The B-tile element this thread stages: k row bk (0..15), 4 consecutive channels from bn.
  const int bk = tid >> 4, bn = (tid & 15) * 4;

  float acc[4][4];
#pragma unroll
  for(int i = 0; i < 4; i++)
#pragma unroll
    for(int j = 0; j < 4; j++) acc[i][j] = 0.0f;

  for(int dy = 0; dy < kY; dy++) {
    for(int dx = 0; dx < kX; dx++) {
      const int iy = ly + dy - padY, ix = lx + dx - padX;
      const bool inb = lvalid && iy >= 0 && iy < g.Y && ix >= 0 && ix < g.X;
      const T* arow = in + ((size_t)lb * g.PB + (size_t)iy * g.RW + ix) * inStride;
      const T* wtap = w + (size_t)(dy * kX + dx) * inC * outC;
      for(int k0 = 0; k0 < inC; k0 += SC_BK) {
#pragma unroll
        for(int q = 0; q < 4; q++) {
          int k = k0 + lk + q;
          sA[lk + q][lr] = (inb && k < inC) ? toF<T>(arow[k]) : 0.0f;
        }
#pragma unroll
        for(int q = 0; q < 4; q++) {
          int k = k0 + bk, c = n0 + bn + q;
          sB[bk][bn + q] = (k < inC && c < outC) ? toF<T>(wtap[(size_t)k * outC + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for(int k = 0; k < SC_BK; k++) {
          float a[4], b[4];
#pragma unroll
          for(int i = 0; i < 4; i++) a[i] = sA[k][ty * 4 + i];
#pragma unroll
          for(int j = 0; j < 4; j++) b[j] = sB[k][tx * 4 + j];
#pragma unroll
          for(int i = 0; i < 4; i++)
#pragma unroll
            for(int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
      }
    }
  }

  // Epilogue
#pragma unroll
  for(int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if(m >= g.rowsPad) continue;
    const int b = min(m / g.PB, g.n - 1);
    const float mk = ep.mask ? ep.mask[m] : 1.0f;
#pragma unroll
    for(int j = 0; j < 4; j++) {
      const int c = n0 + tx * 4 + j;
      if(c >= outC) continue;
      float v = acc[i][j];
      if(ep.biasNC) v += ep.biasNC[(size_t)b * outC + c];
      if(ep.residual) v = (ep.resMask ? v * mk : v) + toF<T>(((const T*)ep.residual)[(size_t)m * ep.resStride + c]);
      if(ep.outRaw && c >= ep.rawC0 && c < ep.rawC1) ((T*)ep.outRaw)[(size_t)m * ep.rawStride + (c - ep.rawC0)] = fromF<T>(v);
      if(ep.outAct && c >= ep.actC0 && c < ep.actC1) {
        const int ca = c - ep.actC0;
        float a = (mk == 1.0f) ? applyActF(v * ep.scale[ca] + ep.bias[ca], ep.act) : 0.0f;
        ((T*)ep.outAct)[(size_t)m * ep.actStride + ca] = fromF<T>(a);
      }
    }
  }
}

cudaError_t launchConvSimt(
  cudaStream_t st, int dt, const void* in, int inStride, int inC, const void* w, int outC, int kY, int kX,
  Geom g, const Epilogue& ep) {
  dim3 grid(g.rowsPad / SC_BM, (outC + SC_BN - 1) / SC_BN);
  KB_DISPATCH_DT(dt, (convSimtKernel<T><<<grid, 256, 0, st>>>((const T*)in, inStride, inC, (const T*)w, outC, kY, kX, g, ep)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Small matmul: one block per row

constexpr int MM_ROWS = 4;
constexpr int MM_KSPLIT = 4;  // the input channels are split over threadIdx.y so that each thread's dependent chain is short

__global__ void matMulSmallKernel(
  const float* __restrict__ in, int inC, const float* __restrict__ w, int outC, const float* __restrict__ bias, int act,
  float* __restrict__ out, int rows, int accumulate) {
  extern __shared__ float sIn[];  // [MM_ROWS][inC], then partial sums [MM_KSPLIT][MM_ROWS][blockDim.x]
  float* sPart = sIn + MM_ROWS * inC;
  const int r0 = blockIdx.x * MM_ROWS;
  const int nr = min(MM_ROWS, rows - r0);
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nthreads = blockDim.x * blockDim.y;
  for(int i = tid; i < MM_ROWS * inC; i += nthreads) {
    const int r = i / inC;
    sIn[i] = r < nr ? in[(size_t)r0 * inC + i] : 0.0f;
  }
  __syncthreads();
  const int kPer = (inC + MM_KSPLIT - 1) / MM_KSPLIT;
  const int k0 = threadIdx.y * kPer, k1 = min(inC, k0 + kPer);
  for(int ocBase = 0; ocBase < outC; ocBase += blockDim.x) {
    const int oc = ocBase + threadIdx.x;
    float s[MM_ROWS];
#pragma unroll
    for(int r = 0; r < MM_ROWS; r++) s[r] = 0.0f;
    if(oc < outC) {
#pragma unroll 8
      for(int ic = k0; ic < k1; ic++) {
        const float wv = w[(size_t)ic * outC + oc];
#pragma unroll
        for(int r = 0; r < MM_ROWS; r++) s[r] = fmaf(sIn[r * inC + ic], wv, s[r]);
      }
    }
#pragma unroll
    for(int r = 0; r < MM_ROWS; r++) sPart[(threadIdx.y * MM_ROWS + r) * blockDim.x + threadIdx.x] = s[r];
    __syncthreads();
    if(threadIdx.y == 0 && oc < outC) {
      const float b = bias ? bias[oc] : 0.0f;
#pragma unroll
      for(int r = 0; r < MM_ROWS; r++) {
        float t = 0.0f;
#pragma unroll
        for(int k = 0; k < MM_KSPLIT; k++) t += sPart[(k * MM_ROWS + r) * blockDim.x + threadIdx.x];
        if(r < nr) {
          float* o = out + (size_t)(r0 + r) * outC + oc;
          const float y = applyActF(t + b, act);
          *o = accumulate ? *o + y : y;
        }
      }
    }
    __syncthreads();
  }
}

cudaError_t launchMatMulSmall(
  cudaStream_t st, const float* in, int inC, const float* w, int outC, const float* bias, int act, float* out, int rows, int accumulate) {
  const int threads = outC >= 128 ? 128 : (outC > 32 ? 64 : 32);
  const size_t smem = (size_t)(MM_ROWS * inC + MM_KSPLIT * MM_ROWS * threads) * sizeof(float);
  matMulSmallKernel<<<(rows + MM_ROWS - 1) / MM_ROWS, dim3(threads, MM_KSPLIT), smem, st>>>(in, inC, w, outC, bias, act, out, rows, accumulate);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Masked global pooling.  grid (n, ceil(C/32)), block (32 channels, 8 point groups).

template <typename T>
__global__ void gpoolKernel(
  const T* __restrict__ in, int inStride, int c0, int C, const float* __restrict__ mask, const float* __restrict__ maskSum,
  float* __restrict__ out, int valueHead, Geom g) {
  const int n = blockIdx.x;
  const int c = blockIdx.y * 32 + threadIdx.x;
  float s = 0.0f, mx = -1.0f;
  if(c < C) {
    for(int p = threadIdx.y; p < g.S; p += blockDim.y) {
      int y = p / g.X, x = p - y * g.X;
      size_t row = (size_t)n * g.PB + (size_t)y * g.RW + x;
      float v = toF<T>(in[row * inStride + c0 + c]);
      s += v;
      mx = fmaxf(mx, v + (mask[row] - 1.0f));
    }
  }
  __shared__ float sSum[8][33], sMax[8][33];
  sSum[threadIdx.y][threadIdx.x] = s;
  sMax[threadIdx.y][threadIdx.x] = mx;
  __syncthreads();
  if(threadIdx.y == 0 && c < C) {
    for(int k = 1; k < blockDim.y; k++) { s += sSum[k][threadIdx.x]; mx = fmaxf(mx, sMax[k][threadIdx.x]); }
    float div = maskSum[n];
    float sq = sqrtf(div);
    float mean = s / div;
    float* o = out + (size_t)n * 3 * C;
    o[c] = mean;
    o[C + c] = mean * (sq - 14.0f) * 0.1f;
    o[2 * C + c] = valueHead ? mean * ((sq - 14.0f) * (sq - 14.0f) * 0.01f - 0.1f) : mx;
  }
}

// Vectorised variant: one block per board, each thread owns 8 adjacent channels (16 bytes) of every k-th point.
template <typename T>
__global__ void __launch_bounds__(256) gpoolVec8Kernel(
  const T* __restrict__ in, int inStride, int c0, int C, const float* __restrict__ mask, const float* __restrict__ maskSum,
  float* __restrict__ out, int valueHead, Geom g) {
  extern __shared__ float sRed[];  // [groups][C] sums then [groups][C] maxima
  const int n = blockIdx.x;
  const int vecs = C / 8;
  const int groups = blockDim.x / vecs;
  const int cg = threadIdx.x % vecs, rg = threadIdx.x / vecs;
  float s[8], mx[8];
#pragma unroll
  for(int j = 0; j < 8; j++) { s[j] = 0.0f; mx[j] = -1.0f; }
  if(rg < groups) {
#pragma unroll 4
    for(int p = rg; p < g.S; p += groups) {
      const int y = p / g.X, x = p - y * g.X;
      const size_t row = (size_t)n * g.PB + (size_t)y * g.RW + x;
      const uint4 v4 = *reinterpret_cast<const uint4*>(in + row * inStride + c0 + cg * 8);
      const T* ve = reinterpret_cast<const T*>(&v4);
      const float mOff = mask[row] - 1.0f;
#pragma unroll
      for(int j = 0; j < 8; j++) {
        const float v = toF<T>(ve[j]);
        s[j] += v;
        mx[j] = fmaxf(mx[j], v + mOff);
      }
    }
#pragma unroll
    for(int j = 0; j < 8; j++) { sRed[rg * C + cg * 8 + j] = s[j]; sRed[(groups + rg) * C + cg * 8 + j] = mx[j]; }
  }
  __syncthreads();
  for(int c = threadIdx.x; c < C; c += blockDim.x) {
    float ss = 0.0f, mm = -1.0f;
    for(int k = 0; k < groups; k++) { ss += sRed[k * C + c]; mm = fmaxf(mm, sRed[(groups + k) * C + c]); }
    const float div = maskSum[n];
    const float sq = sqrtf(div);
    const float mean = ss / div;
    float* o = out + (size_t)n * 3 * C;
    o[c] = mean;
    o[C + c] = mean * (sq - 14.0f) * 0.1f;
    o[2 * C + c] = valueHead ? mean * ((sq - 14.0f) * (sq - 14.0f) * 0.01f - 0.1f) : mm;
  }
}

cudaError_t launchGPool(
  cudaStream_t st, int dt, const void* in, int inStride, int c0, int C, const float* mask, const float* maskSum,
  float* out, int valueHead, Geom g) {
  if(dt != DT_F32 && (C % 8) == 0 && (c0 % 8) == 0 && (inStride % 8) == 0 && C / 8 <= 256 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    const int groups = 256 / (C / 8);
    const size_t smem = (size_t)2 * groups * C * sizeof(float);
    if(dt == DT_F16)
      gpoolVec8Kernel<__half><<<g.n, 256, smem, st>>>((const __half*)in, inStride, c0, C, mask, maskSum, out, valueHead, g);
    else
      gpoolVec8Kernel<__nv_bfloat16><<<g.n, 256, smem, st>>>((const __nv_bfloat16*)in, inStride, c0, C, mask, maskSum, out, valueHead, g);
    return cudaGetLastError();
  }
  dim3 grid(g.n, (C + 31) / 32), block(32, 8);
  KB_DISPATCH_DT(dt, (gpoolKernel<T><<<grid, block, 0, st>>>((const T*)in, inStride, c0, C, mask, maskSum, out, valueHead, g)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Elementwise passes

template <typename TI, typename TO>
__global__ void biasBnActKernel(
  const TI* __restrict__ in, int inStride, const float* __restrict__ biasNC, const float* __restrict__ scale,
  const float* __restrict__ bias, int act, const float* __restrict__ mask, TO* __restrict__ out, int outStride, int C, Geom g) {
  const size_t total = (size_t)g.rowsPad * C;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t m = idx / C;
    int c = (int)(idx - m * C);
    float r = 0.0f;
    if(m < (size_t)g.rows && mask[m] == 1.0f) {
      float v = toF<TI>(in[m * inStride + c]);
      if(biasNC) v += biasNC[(m / g.PB) * C + c];
      r = applyActF(v * scale[c] + bias[c], act);
    }
    out[m * outStride + c] = fromF<TO>(r);
  }
}

// 8 channels (16 bytes) per thread; rows and channel count are multiples of 8 elements.
template <typename T>
__global__ void biasBnActVec8Kernel(
  const T* __restrict__ in, int inStride, const float* __restrict__ biasNC, const float* __restrict__ scale,
  const float* __restrict__ bias, int act, const float* __restrict__ mask, T* __restrict__ out, int outStride, int C, Geom g) {
  const int vecPerRow = C / 8;
  const size_t total = (size_t)g.rowsPad * vecPerRow;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / vecPerRow;
    const int c = (int)(idx - m * vecPerRow) * 8;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if(m < (size_t)g.rows && mask[m] == 1.0f) {
      const uint4 x = *reinterpret_cast<const uint4*>(in + m * inStride + c);
      const T* xe = reinterpret_cast<const T*>(&x);
      T* oe = reinterpret_cast<T*>(&o);
      float v[8];
#pragma unroll
      for(int j = 0; j < 8; j++) v[j] = toF<T>(xe[j]);
      if(biasNC) {
        const float4* bn4 = reinterpret_cast<const float4*>(biasNC + (m / g.PB) * C + c);
        const float4 b0 = bn4[0], b1 = bn4[1];
        v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w; v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
      }
      const float4* s4 = reinterpret_cast<const float4*>(scale + c);
      const float4* b4 = reinterpret_cast<const float4*>(bias + c);
      const float4 s0 = s4[0], s1 = s4[1], c0 = b4[0], c1 = b4[1];
      const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const float bi[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      // reduced-precision output: the fast activation's error is far below the rounding of the result
#pragma unroll
      for(int j = 0; j < 8; j++) oe[j] = fromF<T>(fastAct(fmaf(v[j], sc[j], bi[j]), act));
    }
    *reinterpret_cast<uint4*>(out + m * outStride + c) = o;
  }
}

static int ewGrid(size_t total) {
  size_t b = (total + 255) / 256;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

cudaError_t launchBiasBnAct(
  cudaStream_t st, int dt, const void* in, int inStride, const float* biasNC, const float* scale, const float* bias,
  int act, const float* mask, void* out, int outStride, int C, Geom g) {
  const bool vec = dt != DT_F32 && (C % 8) == 0 && (inStride % 8) == 0 && (outStride % 8) == 0 &&
                   (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  if(vec) {
    int grid = ewGrid((size_t)g.rowsPad * (C / 8));
    if(dt == DT_F16)
      biasBnActVec8Kernel<__half><<<grid, 256, 0, st>>>((const __half*)in, inStride, biasNC, scale, bias, act, mask, (__half*)out, outStride, C, g);
    else
      biasBnActVec8Kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, inStride, biasNC, scale, bias, act, mask, (__nv_bfloat16*)out, outStride, C, g);
    return cudaGetLastError();
  }
  int grid = ewGrid((size_t)g.rowsPad * C);
  KB_DISPATCH_DT(dt, (biasBnActKernel<T, T><<<grid, 256, 0, st>>>((const T*)in, inStride, biasNC, scale, bias, act, mask, (T*)out, outStride, C, g)));
  return cudaGetLastError();
}

cudaError_t launchBnAct(
  cudaStream_t st, int dtIn, const void* in, int inStride, const float* scale, const float* bias, int act,
  const float* mask, int dtOut, void* out, int outStride, int C, Geom g) {
  int grid = ewGrid((size_t)g.rowsPad * C);
  if(dtIn != dtOut && dtIn != DT_F32) return cudaErrorInvalidValue;
  if(dtIn == dtOut) {
    KB_DISPATCH_DT(dtIn, (biasBnActKernel<T, T><<<grid, 256, 0, st>>>((const T*)in, inStride, nullptr, scale, bias, act, mask, (T*)out, outStride, C, g)));
  }
  else {
    KB_DISPATCH_DT(dtOut, (biasBnActKernel<float, T><<<grid, 256, 0, st>>>((const float*)in, inStride, nullptr, scale, bias, act, mask, (T*)out, outStride, C, g)));
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// The middle of a global-pooling block in one launch (eigenbackend.cpp:1188-1211): pooled statistics of the activated gpool
// branch, the 3*Cg -> Cr matmul that turns them into a per-board bias, and the pass that adds that bias to the regular
// branch and applies the next norm + activation + mask.  Everything is per board, so a board's CTAs need nothing from
// other boards: grid (n, GPM_SPLIT); every CTA of a board computes the board's statistics and bias (the second reader of
// the gpool branch hits L2) and then takes its share of the board's rows.
// out[oc] = act(sum_k in[k] * wT[oc][k] + bias[oc]) for oc < outC; in and out in shared memory, all warps take part.
// The weights are stored output-major: a warp takes an output at a time, its lanes stride over k with coalesced loads
// that are all in flight together (a thread-per-output loop over [k][oc] weights has one dependent chain of K
// L2-latency loads per thread, which is what made the separate small matmul launches slow), then reduce by shuffles.
__device__ __forceinline__ void blockMatVecT(const float* in, int K, const float* __restrict__ wT, int outC, const float* __restrict__ bias, int act, float* out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for(int oc0 = warp * 4; oc0 < outC; oc0 += nwarps * 4) {
    float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // rows past the last output are read from the last one (and dropped), so that every load is unconditional and
    // the loads of several k steps can be in flight together
    const float* w0 = wT + (size_t)min(oc0, outC - 1) * K;
    const float* w1 = wT + (size_t)min(oc0 + 1, outC - 1) * K;
    const float* w2 = wT + (size_t)min(oc0 + 2, outC - 1) * K;
    const float* w3 = wT + (size_t)min(oc0 + 3, outC - 1) * K;
#pragma unroll 4
    for(int k = lane; k < K; k += 32) {
      const float x = in[k];
      a[0] = fmaf(x, w0[k], a[0]);
      a[1] = fmaf(x, w1[k], a[1]);
      a[2] = fmaf(x, w2[k], a[2]);
      a[3] = fmaf(x, w3[k], a[3]);
    }
#pragma unroll
    for(int j = 0; j < 4; j++) {
#pragma unroll
      for(int o = 16; o > 0; o >>= 1) a[j] += __shfl_xor_sync(0xffffffffu, a[j], o);
    }
    if(lane < 4 && oc0 + lane < outC) {
      const float t = (lane == 0 ? a[0] : lane == 1 ? a[1] : lane == 2 ? a[2] : a[3]) + (bias ? bias[oc0 + lane] : 0.0f);
      out[oc0 + lane] = applyActF(t, act);
    }
  }
}

constexpr int GPM_SPLIT = 2;
constexpr int GPM_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(GPM_THREADS) gpoolMidVec8Kernel(
  const T* __restrict__ gIn, int gStride, int Cg, const T* __restrict__ rIn, int rStride, int Cr, const float* __restrict__ wT,
  const float* __restrict__ scale, const float* __restrict__ bias, int act, const float* __restrict__ mask,
  const float* __restrict__ maskSum, T* __restrict__ out, int outStride, Geom g) {
  extern __shared__ float sm[];  // [2][groups][Cg] partial sums / maxima, then pooled [3*Cg], then board bias [Cr]
  const int n = blockIdx.x;
  const int vecs = Cg / 8;
  const int groups = GPM_THREADS / vecs;
  float* sPooled = sm + 2 * groups * Cg;
  float* sBias = sPooled + 3 * Cg;
  {
    const int cgv = threadIdx.x % vecs, rg = threadIdx.x / vecs;
    float s[8], mx[8];
#pragma unroll
    for(int j = 0; j < 8; j++) { s[j] = 0.0f; mx[j] = -1.0f; }
    if(rg < groups) {
#pragma unroll 4
      for(int p = rg; p < g.S; p += groups) {
        const int y = p / g.X, x = p - y * g.X;
        const size_t row = (size_t)n * g.PB + (size_t)y * g.RW + x;
        const uint4 v4 = *reinterpret_cast<const uint4*>(gIn + row * gStride + cgv * 8);
        const T* ve = reinterpret_cast<const T*>(&v4);
        const float mOff = mask[row] - 1.0f;
#pragma unroll
        for(int j = 0; j < 8; j++) {
          const float v = toF<T>(ve[j]);
          s[j] += v;
          mx[j] = fmaxf(mx[j], v + mOff);
        }
      }
#pragma unroll
      for(int j = 0; j < 8; j++) { sm[rg * Cg + cgv * 8 + j] = s[j]; sm[(groups + rg) * Cg + cgv * 8 + j] = mx[j]; }
    }
  }
  __syncthreads();
  for(int c = threadIdx.x; c < Cg; c += blockDim.x) {
    float ss = 0.0f, mm = -1.0f;
    for(int k = 0; k < groups; k++) { ss += sm[k * Cg + c]; mm = fmaxf(mm, sm[(groups + k) * Cg + c]); }
    const float div = maskSum[n];
    const float sq = sqrtf(div);
    const float mean = ss / div;
    sPooled[c] = mean;
    sPooled[Cg + c] = mean * (sq - 14.0f) * 0.1f;
    sPooled[2 * Cg + c] = mm;
  }
  __syncthreads();
  blockMatVecT(sPooled, 3 * Cg, wT, Cr, nullptr, KB_ACT_IDENTITY, sBias);
  __syncthreads();
  // this CTA's share of the board's rows (padding rows included: they are written as zeros)
  const int rvecs = Cr / 8;
  const int rowsPer = (g.PB + GPM_SPLIT - 1) / GPM_SPLIT;
  const int r0 = blockIdx.y * rowsPer, r1 = min(g.PB, r0 + rowsPer);
  const int total = (r1 - r0) * rvecs;
  constexpr int U = 4;
  for(int base = threadIdx.x; base < total; base += blockDim.x * U) {
    uint4 xs[U];
    float mk[U];
#pragma unroll
    for(int u = 0; u < U; u++) {
      const int idx = base + u * blockDim.x;
      const int rr = min(idx, total - 1) / rvecs;
      const int c = (min(idx, total - 1) - rr * rvecs) * 8;
      const size_t m = (size_t)n * g.PB + r0 + rr;
      mk[u] = mask[m];
      xs[u] = *reinterpret_cast<const uint4*>(rIn + m * rStride + c);
    }
#pragma unroll
    for(int u = 0; u < U; u++) {
    const int idx = base + u * blockDim.x;
    if(idx >= total) break;
    const int rr = idx / rvecs;
    const int c = (idx - rr * rvecs) * 8;
    const size_t m = (size_t)n * g.PB + r0 + rr;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if(mk[u] == 1.0f) {
      const uint4 x = xs[u];
      const T* xe = reinterpret_cast<const T*>(&x);
      T* oe = reinterpret_cast<T*>(&o);
      const float4* s4 = reinterpret_cast<const float4*>(scale + c);
      const float4* b4 = reinterpret_cast<const float4*>(bias + c);
      const float4 s0 = s4[0], s1 = s4[1], c0 = b4[0], c1 = b4[1];
      const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const float bi[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
      for(int j = 0; j < 8; j++) oe[j] = fromF<T>(fastAct(fmaf(toF<T>(xe[j]) + sBias[c + j], sc[j], bi[j]), act));
    }
    *reinterpret_cast<uint4*>(out + m * outStride + c) = o;
    }
  }
}

bool gpoolMidEligible(int dt, int Cg, int gStride, int Cr, int rStride, int outStride) {
  return dt != DT_F32 && (Cg % 8) == 0 && (Cr % 8) == 0 && (gStride % 8) == 0 && (rStride % 8) == 0 && (outStride % 8) == 0 &&
         Cg / 8 <= GPM_THREADS && Cg >= 8;
}

cudaError_t launchGPoolMid(
  cudaStream_t st, int dt, const void* gIn, int gStride, int Cg, const void* rIn, int rStride, int Cr, const float* w,
  const float* scale, const float* bias, int act, const float* mask, const float* maskSum, void* out, int outStride, Geom g) {
  if(!gpoolMidEligible(dt, Cg, gStride, Cr, rStride, outStride)) return cudaErrorInvalidValue;
  const int groups = GPM_THREADS / (Cg / 8);
  const size_t smem = (size_t)(2 * groups * Cg + 3 * Cg + Cr) * sizeof(float);
  const dim3 grid(g.n, GPM_SPLIT);
  if(dt == DT_F16)
    gpoolMidVec8Kernel<__half><<<grid, GPM_THREADS, smem, st>>>((const __half*)gIn, gStride, Cg, (const __half*)rIn, rStride, Cr, w, scale, bias, act, mask, maskSum, (__half*)out, outStride, g);
  else
    gpoolMidVec8Kernel<__nv_bfloat16><<<grid, GPM_THREADS, smem, st>>>((const __nv_bfloat16*)gIn, gStride, Cg, (const __nv_bfloat16*)rIn, rStride, Cr, w, scale, bias, act, mask, maskSum, (__nv_bfloat16*)out, outStride, g);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Head outputs: one thread per board point.

template <typename T>
__global__ void headFinalKernel(
  const T* __restrict__ pAct, int pStride, int P1, const float* __restrict__ w2, int policyC, const T* __restrict__ vAct,
  int vStride, int v0, int V1, const float* __restrict__ wOwn, const int32_t* __restrict__ symmetry,
  float* __restrict__ policy, float* __restrict__ ownership, Geom g) {
  extern __shared__ float sW[];  // w2 [P1][policyC] then wOwn [V1]
  for(int i = threadIdx.x; i < P1 * policyC; i += blockDim.x) sW[i] = w2[i];
  for(int i = threadIdx.x; i < V1; i += blockDim.x) sW[P1 * policyC + i] = wOwn[i];
  __syncthreads();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if(idx >= g.n * g.S) return;
  const int n = idx / g.S, p = idx - n * g.S;
  const int h = p / g.X, w = p - h * g.X;
  const size_t row = (size_t)n * g.PB + (size_t)h * g.RW + w;
  int h2, w2p;
  symMap(symmetry ? symmetry[n] : 0, true, g.Y, g.X, h, w, h2, w2p);
  const size_t outPos = (size_t)n * g.S + (size_t)h2 * g.X + w2p;
  if(policy) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const T* pr = pAct + row * pStride;
    if(sizeof(T) == 2 && (P1 % 8) == 0 && (pStride % 8) == 0 && (reinterpret_cast<uintptr_t>(pAct) & 15) == 0) {
      // 8 channels per 16-byte load
      for(int c8 = 0; c8 < P1; c8 += 8) {
        const uint4 x = *reinterpret_cast<const uint4*>(pr + c8);
        const T* xe = reinterpret_cast<const T*>(&x);
#pragma unroll
        for(int j = 0; j < 8; j++) {
          const float v = toF<T>(xe[j]);
          for(int k = 0; k < policyC && k < 4; k++) acc[k] = fmaf(v, sW[(c8 + j) * policyC + k], acc[k]);
        }
      }
    }
    else {
      for(int c = 0; c < P1; c++) {
        float v = toF<T>(pr[c]);
        for(int k = 0; k < policyC && k < 4; k++) acc[k] = fmaf(v, sW[c * policyC + k], acc[k]);
      }
    }
    for(int k = 0; k < policyC && k < 4; k++) policy[outPos * policyC + k] = acc[k];
  }
  if(ownership) {
    float o = 0.0f;
    const T* vr = vAct + row * vStride + v0;
    const float* wo = sW + P1 * policyC;
    if(sizeof(T) == 2 && (V1 % 8) == 0 && (vStride % 8) == 0 && (v0 % 8) == 0 && (reinterpret_cast<uintptr_t>(vAct) & 15) == 0) {
      for(int c8 = 0; c8 < V1; c8 += 8) {
        const uint4 x = *reinterpret_cast<const uint4*>(vr + c8);
        const T* xe = reinterpret_cast<const T*>(&x);
#pragma unroll
        for(int j = 0; j < 8; j++) o = fmaf(toF<T>(xe[j]), wo[c8 + j], o);
      }
    }
    else {
      for(int c = 0; c < V1; c++) o = fmaf(toF<T>(vr[c]), wo[c], o);
    }
    ownership[outPos] = o;
  }
}

cudaError_t launchHeadFinal(
  cudaStream_t st, int dt, const void* pAct, int pStride, int P1, const float* w2, int policyC, const void* vAct,
  int vStride, int v0, int V1, const float* wOwn, const int32_t* symmetry, float* policy, float* ownership, Geom g) {
  if(policyC > 4) return cudaErrorInvalidValue;
  int total = g.n * g.S;
  size_t smem = ((size_t)P1 * policyC + V1) * sizeof(float);
  KB_DISPATCH_DT(dt, (headFinalKernel<T><<<(total + 127) / 128, 128, smem, st>>>(
    (const T*)pAct, pStride, P1, w2, policyC, (const T*)vAct, vStride, v0, V1, wOwn, symmetry, policy, ownership, g)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Everything of the heads after their first convolutions, one CTA per board (eigenbackend.cpp:1975-2025, 2063-2103): the two
// poolings, the policy bias, the pass logits, the value MLP, and per board point the policy's norm + activation and
// final 1x1 convolution and the ownership convolution, written in the caller's frame (inverse board symmetry).

constexpr int HT_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(HT_THREADS) headsTailKernel(const HeadsTailArgs a, Geom g) {
  extern __shared__ float sm[];
  const int n = blockIdx.x;
  const int GV = a.G1 + a.V1;
  const int vecs = GV / 8;
  const int groups = HT_THREADS / vecs;
  float* sPart = sm;                                  // [2][groups][GV]
  float* sPoolG = sPart + 2 * groups * GV;            // [3*G1]
  float* sPoolV = sPoolG + 3 * a.G1;                  // [3*V1]
  float* sPBias = sPoolV + 3 * a.V1;                  // [P1]
  float* sHidden = sPBias + a.P1;                     // [passH]
  float* sV2 = sHidden + (a.passH > 0 ? a.passH : 1); // [V2]
  float* sSmall = sV2 + a.V2;                         // pass [Pc], value [Vc], score [Sv]
  float* sW2 = sSmall + a.Pc + a.Vc + a.Sv;           // [P1][Pc]
  float* sWOwn = sW2 + a.P1 * a.Pc;                   // [V1]
  float* sScale = sWOwn + a.V1;                       // [P1] then bias [P1]
  for(int i = threadIdx.x; i < a.P1 * a.Pc; i += blockDim.x) sW2[i] = a.w2[i];
  for(int i = threadIdx.x; i < a.V1; i += blockDim.x) sWOwn[i] = a.wOwn[i];
  for(int i = threadIdx.x; i < a.P1; i += blockDim.x) { sScale[i] = a.pScale[i]; sScale[a.P1 + i] = a.pBias[i]; }
  const T* gv = static_cast<const T*>(a.gv);
  const T* praw = static_cast<const T*>(a.pRaw);
  {
    const int cv = threadIdx.x % vecs, rg = threadIdx.x / vecs;
    float s[8], mx[8];
#pragma unroll
    for(int j = 0; j < 8; j++) { s[j] = 0.0f; mx[j] = -1.0f; }
    if(rg < groups) {
#pragma unroll 2
      for(int p = rg; p < g.S; p += groups) {
        const int y = p / g.X, x = p - y * g.X;
        const size_t row = (size_t)n * g.PB + (size_t)y * g.RW + x;
        const uint4 v4 = *reinterpret_cast<const uint4*>(gv + row * GV + cv * 8);
        const T* ve = reinterpret_cast<const T*>(&v4);
        const float mOff = a.mask[row] - 1.0f;
#pragma unroll
        for(int j = 0; j < 8; j++) {
          const float v = toF<T>(ve[j]);
          s[j] += v;
          mx[j] = fmaxf(mx[j], v + mOff);
        }
      }
#pragma unroll
      for(int j = 0; j < 8; j++) { sPart[rg * GV + cv * 8 + j] = s[j]; sPart[(groups + rg) * GV + cv * 8 + j] = mx[j]; }
    }
  }
  __syncthreads();
  for(int c = threadIdx.x; c < GV; c += blockDim.x) {
    float ss = 0.0f, mm = -1.0f;
    for(int k = 0; k < groups; k++) { ss += sPart[k * GV + c]; mm = fmaxf(mm, sPart[(groups + k) * GV + c]); }
    const float div = a.maskSum[n];
    const float sq = sqrtf(div);
    const float mean = ss / div;
    if(c < a.G1) {
      sPoolG[c] = mean; sPoolG[a.G1 + c] = mean * (sq - 14.0f) * 0.1f; sPoolG[2 * a.G1 + c] = mm;
    }
    else {
      const int cc = c - a.G1;
      sPoolV[cc] = mean; sPoolV[a.V1 + cc] = mean * (sq - 14.0f) * 0.1f; sPoolV[2 * a.V1 + cc] = mean * ((sq - 14.0f) * (sq - 14.0f) * 0.01f - 0.1f);
    }
  }
  __syncthreads();
  blockMatVecT(sPoolG, 3 * a.G1, a.wGB, a.P1, nullptr, KB_ACT_IDENTITY, sPBias);
  if(a.passH > 0) blockMatVecT(sPoolG, 3 * a.G1, a.wPass, a.passH, a.bPass, a.passAct, sHidden);
  else blockMatVecT(sPoolG, 3 * a.G1, a.wPass, a.Pc, nullptr, KB_ACT_IDENTITY, sSmall);
  blockMatVecT(sPoolV, 3 * a.V1, a.wV2, a.V2, a.bV2, a.v2Act, sV2);
  __syncthreads();
  if(a.passH > 0) blockMatVecT(sHidden, a.passH, a.wPass2, a.Pc, nullptr, KB_ACT_IDENTITY, sSmall);
  blockMatVecT(sV2, a.V2, a.wV3, a.Vc, a.bV3, KB_ACT_IDENTITY, sSmall + a.Pc);
  blockMatVecT(sV2, a.V2, a.wSV, a.Sv, a.bSV, KB_ACT_IDENTITY, sSmall + a.Pc + a.Vc);
  __syncthreads();
  for(int i = threadIdx.x; i < a.Pc; i += blockDim.x) a.outPass[(size_t)n * a.Pc + i] = sSmall[i];
  for(int i = threadIdx.x; i < a.Vc; i += blockDim.x) a.outValue[(size_t)n * a.Vc + i] = sSmall[a.Pc + i];
  for(int i = threadIdx.x; i < a.Sv; i += blockDim.x) a.outScore[(size_t)n * a.Sv + i] = sSmall[a.Pc + a.Vc + i];
  const int sym = a.symmetry ? a.symmetry[n] : 0;
  for(int p = threadIdx.x; p < g.S; p += blockDim.x) {
    const int h = p / g.X, w = p - h * g.X;
    const size_t row = (size_t)n * g.PB + (size_t)h * g.RW + w;
    int h2, w2p;
    symMap(sym, true, g.Y, g.X, h, w, h2, w2p);
    const size_t outPos = (size_t)n * g.S + (size_t)h2 * g.X + w2p;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if(a.mask[row] == 1.0f) {
      const T* pr = praw + row * a.P1;
      for(int c8 = 0; c8 < a.P1; c8 += 8) {
        const uint4 x = *reinterpret_cast<const uint4*>(pr + c8);
        const T* xe = reinterpret_cast<const T*>(&x);
#pragma unroll
        for(int j = 0; j < 8; j++) {
          const int c = c8 + j;
          // the activated value passes through the storage type, as it does where this tensor is written out
          const float v = toF<T>(fromF<T>(fastAct(fmaf(toF<T>(xe[j]) + sPBias[c], sScale[c], sScale[a.P1 + c]), a.pAct)));
          for(int k = 0; k < a.Pc && k < 4; k++) acc[k] = fmaf(v, sW2[c * a.Pc + k], acc[k]);
        }
      }
    }
    for(int k = 0; k < a.Pc && k < 4; k++) a.outPolicy[outPos * a.Pc + k] = acc[k];
    float o = 0.0f;
    const T* vr = gv + row * GV + a.G1;
    for(int c8 = 0; c8 < a.V1; c8 += 8) {
      const uint4 x = *reinterpret_cast<const uint4*>(vr + c8);
      const T* xe = reinterpret_cast<const T*>(&x);
#pragma unroll
      for(int j = 0; j < 8; j++) o = fmaf(toF<T>(xe[j]), sWOwn[c8 + j], o);
    }
    a.outOwnership[outPos] = o;
  }
}

bool headsTailEligible(int dt, const HeadsTailArgs& a) {
  const int GV = a.G1 + a.V1;
  return dt != DT_F32 && (a.P1 % 8) == 0 && (a.G1 % 8) == 0 && (a.V1 % 8) == 0 && a.Pc >= 1 && a.Pc <= 4 && GV / 8 <= HT_THREADS &&
         a.P1 <= 512 && a.V2 <= 4096 && a.passH <= 4096;
}

cudaError_t launchHeadsTail(cudaStream_t st, int dt, const HeadsTailArgs& a, Geom g) {
  if(!headsTailEligible(dt, a)) return cudaErrorInvalidValue;
  const int GV = a.G1 + a.V1;
  const int groups = HT_THREADS / (GV / 8);
  const size_t floats = (size_t)2 * groups * GV + 3 * a.G1 + 3 * a.V1 + a.P1 + (a.passH > 0 ? a.passH : 1) + a.V2 + a.Pc + a.Vc + a.Sv +
                        (size_t)a.P1 * a.Pc + a.V1 + 2 * a.P1;
  const size_t smem = floats * sizeof(float);
  if(smem > 200 * 1024) return cudaErrorInvalidValue;
  if(dt == DT_F16) {
    if(smem > 48 * 1024) cudaFuncSetAttribute(headsTailKernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    headsTailKernel<__half><<<g.n, HT_THREADS, smem, st>>>(a, g);
  }
  else {
    if(smem > 48 * 1024) cudaFuncSetAttribute(headsTailKernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    headsTailKernel<__nv_bfloat16><<<g.n, HT_THREADS, smem, st>>>(a, g);
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Layout conversion for single-layer tests

template <typename T>
__global__ void toPaddedKernel(const float* __restrict__ src, int C, T* __restrict__ dst, int dstStride, Geom g) {
  const size_t total = (size_t)g.n * g.S * C;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t p = idx / C;
    int c = (int)(idx - p * C);
    int n = (int)(p / g.S), q = (int)(p - (size_t)n * g.S);
    int y = q / g.X, x = q - y * g.X;
    dst[((size_t)n * g.PB + (size_t)y * g.RW + x) * dstStride + c] = fromF<T>(src[idx]);
  }
}
template <typename T>
__global__ void fromPaddedKernel(const T* __restrict__ src, int srcStride, int C, float* __restrict__ dst, Geom g) {
  const size_t total = (size_t)g.n * g.S * C;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t p = idx / C;
    int c = (int)(idx - p * C);
    int n = (int)(p / g.S), q = (int)(p - (size_t)n * g.S);
    int y = q / g.X, x = q - y * g.X;
    dst[idx] = toF<T>(src[((size_t)n * g.PB + (size_t)y * g.RW + x) * srcStride + c]);
  }
}
__global__ void maskToPaddedKernel(const float* __restrict__ src, float* __restrict__ mask, float* __restrict__ maskSum, Geom g) {
  const int n = blockIdx.x;
  float s = 0.0f;
  for(int p = threadIdx.x; p < g.S; p += blockDim.x) {
    int y = p / g.X, x = p - y * g.X;
    float v = src[(size_t)n * g.S + p];
    mask[(size_t)n * g.PB + (size_t)y * g.RW + x] = v;
    s += v;
  }
  __shared__ float red[32];
  for(int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if(threadIdx.x < 32) {
    float v = (threadIdx.x < (blockDim.x + 31) / 32) ? red[threadIdx.x] : 0.0f;
    for(int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if(threadIdx.x == 0) maskSum[n] = v;
  }
}

cudaError_t launchToPadded(cudaStream_t st, int dt, const float* src, int C, void* dst, int dstStride, Geom g) {
  int grid = ewGrid((size_t)g.n * g.S * C);
  KB_DISPATCH_DT(dt, (toPaddedKernel<T><<<grid, 256, 0, st>>>(src, C, (T*)dst, dstStride, g)));
  return cudaGetLastError();
}
cudaError_t launchFromPadded(cudaStream_t st, int dt, const void* src, int srcStride, int C, float* dst, Geom g) {
  int grid = ewGrid((size_t)g.n * g.S * C);
  KB_DISPATCH_DT(dt, (fromPaddedKernel<T><<<grid, 256, 0, st>>>((const T*)src, srcStride, C, dst, g)));
  return cudaGetLastError();
}
cudaError_t launchMaskToPadded(cudaStream_t st, const float* src, float* mask, float* maskSum, Geom g) {
  maskToPaddedKernel<<<g.n, 128, 0, st>>>(src, mask, maskSum, g);
  return cudaGetLastError();
}

}  // namespace kb
