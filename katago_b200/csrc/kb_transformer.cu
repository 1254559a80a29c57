// CUDA-core kernels of the transformer trunk blocks: RMS norms, rotary embedding, masked attention over the
// board points, SwiGLU.  The projections (Q/K/V, output, FFN) are 1x1 convolutions and use the convolution
// kernels.  All of these are memory-bound except attention, which here is a straightforward shared-memory
// implementation on CUDA cores (one block per board, head and 32-query slice).
#include "kb_kernels.cuh"
#include "kb_act.cuh"
#include "../../include/kb_modelblob.h"

namespace kb {

template <typename T> __device__ __forceinline__ float tToF(T v);
template <> __device__ __forceinline__ float tToF<float>(float v) { return v; }
template <> __device__ __forceinline__ float tToF<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float tToF<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T fToT(float v);
template <> __device__ __forceinline__ float fToT<float>(float v) { return v; }
template <> __device__ __forceinline__ __half fToT<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 fToT<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

#define KBT_DISPATCH_DT(dt, EXPR)                                  \
  switch(dt) {                                                     \
    case DT_F32: { using T = float; EXPR; break; }                 \
    case DT_F16: { using T = __half; EXPR; break; }                \
    case DT_BF16: { using T = __nv_bfloat16; EXPR; break; }        \
    default: return cudaErrorInvalidValue;                         \
  }

__device__ __forceinline__ float warpSum(float v) {
  for(int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warpMax(float v) {
  for(int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
// RMS norm: one warp per row

template <typename T>
__global__ void rmsNormKernel(
  const T* __restrict__ in, int inStride, const float* __restrict__ gamma, const float* __restrict__ beta, float eps, int silu,
  const float* __restrict__ mask, const float* __restrict__ boardScale, T* __restrict__ out, int outStride, int C, Geom g) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if(row >= g.rowsPad) return;
  T* o = out + (size_t)row * outStride;
  if(row >= g.rows || mask[row] == 0.0f) {
    for(int c = lane; c < C; c += 32) o[c] = fToT<T>(0.0f);
    return;
  }
  const T* x = in + (size_t)row * inStride;
  float rms;
  if(boardScale) rms = boardScale[row / g.PB];
  else {
    float ss = 0.0f;
    for(int c = lane; c < C; c += 32) { float v = tToF<T>(x[c]); ss += v * v; }
    ss = warpSum(ss);
    rms = 1.0f / sqrtf(ss / (float)C + eps);
  }
  for(int c = lane; c < C; c += 32) {
    float v = tToF<T>(x[c]) * rms * gamma[c];
    if(beta) v += beta[c];
    if(silu) v = v / (1.0f + expf(-v));
    o[c] = fToT<T>(v);
  }
}

// The same for 16-bit element types with C a multiple of 8 and at most 512: a lane keeps its one or two 8-channel
// chunks of the row in registers between the sum of squares and the scaling, and memory sees 16-byte accesses only.
// The arithmetic per element is that of rmsNormKernel except for the SiLU, see below.
template <typename T>
__global__ void rmsNormVec8Kernel(
  const T* __restrict__ in, int inStride, const float* __restrict__ gamma, const float* __restrict__ beta, float eps, int silu,
  const float* __restrict__ mask, const float* __restrict__ boardScale, T* __restrict__ out, int outStride, int C, Geom g) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if(row >= g.rowsPad) return;
  const int chunks = C >> 3;
  T* o = out + (size_t)row * outStride;
  if(row >= g.rows || mask[row] == 0.0f) {
    for(int j = lane; j < chunks; j += 32) *reinterpret_cast<uint4*>(o + 8 * j) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const T* x = in + (size_t)row * inStride;
  uint4 raw[2];
  float ss = 0.0f;
#pragma unroll
  for(int k = 0; k < 2; k++) {
    const int j = lane + 32 * k;
    raw[k] = make_uint4(0u, 0u, 0u, 0u);
    if(j < chunks) {
      raw[k] = *reinterpret_cast<const uint4*>(x + 8 * j);
      const T* e = reinterpret_cast<const T*>(&raw[k]);
#pragma unroll
      for(int i = 0; i < 8; i++) { const float v = tToF<T>(e[i]); ss += v * v; }
    }
  }
  float rms;
  if(boardScale) rms = boardScale[row / g.PB];
  else rms = 1.0f / sqrtf(warpSum(ss) / (float)C + eps);
#pragma unroll
  for(int k = 0; k < 2; k++) {
    const int j = lane + 32 * k;
    if(j >= chunks) continue;
    const T* e = reinterpret_cast<const T*>(&raw[k]);
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + 8 * j), g1 = *reinterpret_cast<const float4*>(gamma + 8 * j + 4);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    float bb[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if(beta) {
      const float4 b0 = *reinterpret_cast<const float4*>(beta + 8 * j), b1 = *reinterpret_cast<const float4*>(beta + 8 * j + 4);
      bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
    }
    uint4 res;
    T* r = reinterpret_cast<T*>(&res);
#pragma unroll
    for(int i = 0; i < 8; i++) {
      float v = tToF<T>(e[i]) * rms * gg[i];
      if(beta) v += bb[i];
      // the special-function form the convolution epilogues use (kb_act.cuh): its error is far below the rounding of
      // the 16-bit result, and the exact expf + division made this kernel compute-bound
      if(silu) v = v * rcpApprox(1.0f + ex2Approx(v * -1.4426950408889634f));
      r[i] = fToT<T>(v);
    }
    *reinterpret_cast<uint4*>(o + 8 * j) = res;
  }
}

static bool rmsNormVec8Ok(int dt, const void* in, int inStride, const float* gamma, const float* beta, const void* out, int outStride, int C) {
  return dt != DT_F32 && (C % 8) == 0 && C <= 512 && (inStride % 8) == 0 && (outStride % 8) == 0 &&
         (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(gamma) & 15) == 0 && (beta == nullptr || (reinterpret_cast<uintptr_t>(beta) & 15) == 0);
}

cudaError_t launchRmsNorm(
  cudaStream_t st, int dt, const void* in, int inStride, const float* gamma, const float* beta, float eps, int silu,
  const float* mask, void* out, int outStride, int C, Geom g) {
  const int warps = 8;
  if(rmsNormVec8Ok(dt, in, inStride, gamma, beta, out, outStride, C)) {
    if(dt == DT_F16)
      rmsNormVec8Kernel<__half><<<(g.rowsPad + warps - 1) / warps, warps * 32, 0, st>>>(
        (const __half*)in, inStride, gamma, beta, eps, silu, mask, nullptr, (__half*)out, outStride, C, g);
    else
      rmsNormVec8Kernel<__nv_bfloat16><<<(g.rowsPad + warps - 1) / warps, warps * 32, 0, st>>>(
        (const __nv_bfloat16*)in, inStride, gamma, beta, eps, silu, mask, nullptr, (__nv_bfloat16*)out, outStride, C, g);
    return cudaGetLastError();
  }
  KBT_DISPATCH_DT(dt, (rmsNormKernel<T><<<(g.rowsPad + warps - 1) / warps, warps * 32, 0, st>>>(
    (const T*)in, inStride, gamma, beta, eps, silu, mask, nullptr, (T*)out, outStride, C, g)));
  return cudaGetLastError();
}

// per-board 1/rms over all on-board points and channels: one block per board
template <typename T>
__global__ void boardRmsKernel(const T* __restrict__ in, int inStride, const float* __restrict__ mask, float eps, float* __restrict__ outScale, int C, Geom g) {
  const int n = blockIdx.x;
  float ss = 0.0f, cnt = 0.0f;
  for(int p = threadIdx.x >> 5; p < g.S; p += (blockDim.x >> 5)) {
    const int y = p / g.X, x = p - y * g.X;
    const size_t row = (size_t)n * g.PB + (size_t)y * g.RW + x;
    if(mask[row] == 0.0f) continue;
    const T* xr = in + row * inStride;
    for(int c = threadIdx.x & 31; c < C; c += 32) { float v = tToF<T>(xr[c]); ss += v * v; }
    if((threadIdx.x & 31) == 0) cnt += 1.0f;
  }
  __shared__ float sS[32], sC[32];
  ss = warpSum(ss); cnt = warpSum(cnt);
  if((threadIdx.x & 31) == 0) { sS[threadIdx.x >> 5] = ss; sC[threadIdx.x >> 5] = cnt; }
  __syncthreads();
  if(threadIdx.x < 32) {
    float a = threadIdx.x < (blockDim.x >> 5) ? sS[threadIdx.x] : 0.0f;
    float b = threadIdx.x < (blockDim.x >> 5) ? sC[threadIdx.x] : 0.0f;
    a = warpSum(a); b = warpSum(b);
    if(threadIdx.x == 0) outScale[n] = 1.0f / sqrtf(a / (b * (float)C) + eps);
  }
}

cudaError_t launchSpatialRmsNorm(
  cudaStream_t st, int dt, const void* in, int inStride, const float* gamma, const float* beta, float eps, int silu,
  const float* mask, void* out, int outStride, int C, float* scratch, Geom g) {
  const int warps = 8;
  KBT_DISPATCH_DT(dt, (boardRmsKernel<T><<<g.n, 256, 0, st>>>((const T*)in, inStride, mask, eps, scratch, C, g)));
  cudaError_t e = cudaGetLastError();
  if(e != cudaSuccess) return e;
  KBT_DISPATCH_DT(dt, (rmsNormKernel<T><<<(g.rowsPad + warps - 1) / warps, warps * 32, 0, st>>>(
    (const T*)in, inStride, gamma, beta, eps, silu, mask, scratch, (T*)out, outStride, C, g)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding

template <typename T>
__global__ void ropeKernel(
  T* __restrict__ buf, int stride, int c0, int heads, int dim, const float* __restrict__ cosT, const float* __restrict__ sinT,
  int tableHeads, Geom g) {
  const int pairs = dim / 2;
  const size_t total = (size_t)g.n * g.S * heads * pairs;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int p = (int)(idx % pairs);
    size_t r = idx / pairs;
    const int h = (int)(r % heads);
    r /= heads;
    const int xy = (int)(r % g.S), n = (int)(r / g.S);
    const int y = xy / g.X, x = xy - y * g.X;
    T* e = buf + ((size_t)n * g.PB + (size_t)y * g.RW + x) * stride + c0 + h * dim + 2 * p;
    const int th = h * tableHeads / heads;
    const size_t t = ((size_t)th * pairs + p) * g.S + xy;
    const float c = cosT[t], s = sinT[t];
    const float x0 = tToF<T>(e[0]), x1 = tToF<T>(e[1]);
    e[0] = fToT<T>(x0 * c - x1 * s);
    e[1] = fToT<T>(x0 * s + x1 * c);
  }
}

// 8 channels (4 pairs) per thread
template <typename T>
__global__ void ropeVec8Kernel(
  T* __restrict__ buf, int stride, int c0, int heads, int dim, const float* __restrict__ cosT, const float* __restrict__ sinT,
  int tableHeads, Geom g) {
  const int pairs = dim / 2, vecsPerHead = dim / 8;
  const size_t total = (size_t)g.n * g.S * heads * vecsPerHead;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vecsPerHead);
    size_t r = idx / vecsPerHead;
    const int h = (int)(r % heads);
    r /= heads;
    const int xy = (int)(r % g.S), n = (int)(r / g.S);
    const int y = xy / g.X, x = xy - y * g.X;
    T* e = buf + ((size_t)n * g.PB + (size_t)y * g.RW + x) * stride + c0 + h * dim + v * 8;
    uint4 val = *reinterpret_cast<uint4*>(e);
    T* ve = reinterpret_cast<T*>(&val);
    const int th = h * tableHeads / heads;
#pragma unroll
    for(int j = 0; j < 4; j++) {
      const size_t t = ((size_t)th * pairs + v * 4 + j) * g.S + xy;
      const float c = cosT[t], s = sinT[t];
      const float x0 = tToF<T>(ve[2 * j]), x1 = tToF<T>(ve[2 * j + 1]);
      ve[2 * j] = fToT<T>(x0 * c - x1 * s);
      ve[2 * j + 1] = fToT<T>(x0 * s + x1 * c);
    }
    *reinterpret_cast<uint4*>(e) = val;
  }
}

cudaError_t launchRope(
  cudaStream_t st, int dt, void* buf, int stride, int c0, int heads, int dim, const float* cosT, const float* sinT,
  int tableHeads, Geom g) {
  if(dt != DT_F32 && (dim % 8) == 0 && (stride % 8) == 0 && (c0 % 8) == 0 && (reinterpret_cast<uintptr_t>(buf) & 15) == 0) {
    const size_t totalV = (size_t)g.n * g.S * heads * (dim / 8);
    int gridV = (int)((totalV + 255) / 256);
    if(gridV > 148 * 32) gridV = 148 * 32;
    if(dt == DT_F16) ropeVec8Kernel<__half><<<gridV, 256, 0, st>>>((__half*)buf, stride, c0, heads, dim, cosT, sinT, tableHeads, g);
    else ropeVec8Kernel<__nv_bfloat16><<<gridV, 256, 0, st>>>((__nv_bfloat16*)buf, stride, c0, heads, dim, cosT, sinT, tableHeads, g);
    return cudaGetLastError();
  }
  const size_t total = (size_t)g.n * g.S * heads * (dim / 2);
  int grid = (int)((total + 255) / 256);
  if(grid > 148 * 16) grid = 148 * 16;
  KBT_DISPATCH_DT(dt, (ropeKernel<T><<<grid, 256, 0, st>>>((T*)buf, stride, c0, heads, dim, cosT, sinT, tableHeads, g)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Attention.  grid (ceil(S/32), n*heads), 256 threads = 8 warps, each warp owns 4 of the block's 32 queries.
// K and V of the (board, kv head) live in shared memory as fp32 with an odd row pitch; scores of the warp's
// current query live in shared memory too.

template <typename T>
__global__ void __launch_bounds__(256) attentionKernel(
  const T* __restrict__ qkv, int stride, int qOff, int kOff, int vOff, int heads, int kvHeads, int dq, int dv,
  const float* __restrict__ mask, T* __restrict__ out, int outStride, Geom g, const float* __restrict__ relBias, int relY, int relX) {
  extern __shared__ float sm[];
  const int S = g.S;
  const int kp = dq + 1, vp = dv + 1;
  float* sK = sm;                      // [S][kp]
  float* sV = sK + (size_t)S * kp;     // [S][vp]
  float* sMask = sV + (size_t)S * vp;  // [S]
  float* sP = sMask + S;               // [8][S]
  float* sQ = sP + 8 * S;              // [8][dq]
  const int n = blockIdx.y / heads, h = blockIdx.y % heads;
  const int kvh = h / (heads / kvHeads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t boardRow = (size_t)n * g.PB;
  for(int idx = threadIdx.x; idx < S * dq; idx += blockDim.x) {
    const int p = idx / dq, d = idx - p * dq;
    const int y = p / g.X, x = p - y * g.X;
    sK[p * kp + d] = tToF<T>(qkv[(boardRow + (size_t)y * g.RW + x) * stride + kOff + kvh * dq + d]);
  }
  for(int idx = threadIdx.x; idx < S * dv; idx += blockDim.x) {
    const int p = idx / dv, d = idx - p * dv;
    const int y = p / g.X, x = p - y * g.X;
    sV[p * vp + d] = tToF<T>(qkv[(boardRow + (size_t)y * g.RW + x) * stride + vOff + kvh * dv + d]);
  }
  for(int p = threadIdx.x; p < S; p += blockDim.x) {
    const int y = p / g.X, x = p - y * g.X;
    sMask[p] = mask[boardRow + (size_t)y * g.RW + x];
  }
  __syncthreads();
  const float scale = 1.0f / sqrtf((float)dq);
  float* myP = sP + warp * S;
  float* myQ = sQ + warp * dq;
  for(int qi = blockIdx.x * 32 + warp; qi < min(S, blockIdx.x * 32 + 32); qi += 8) {
    const int y = qi / g.X, x = qi - y * g.X;
    const size_t row = boardRow + (size_t)y * g.RW + x;
    T* o = out + row * outStride + h * dv;
    if(sMask[qi] == 0.0f) {
      for(int d = lane; d < dv; d += 32) o[d] = fToT<T>(0.0f);
      continue;
    }
    for(int d = lane; d < dq; d += 32) myQ[d] = tToF<T>(qkv[row * stride + qOff + h * dq + d]);
    __syncwarp();
    float mx = -1e30f;
    for(int k = lane; k < S; k += 32) {
      float s = -1e30f;
      if(sMask[k] != 0.0f) {
        const float* kr = sK + k * kp;
        float dot = 0.0f;
        for(int d = 0; d < dq; d++) dot = fmaf(myQ[d], kr[d], dot);
        s = dot * scale;
        if(relBias) {
          const int ky = k / g.X, kx = k - ky * g.X;
          s += relBias[((size_t)h * (2 * relY - 1) + (ky - y + relY - 1)) * (2 * relX - 1) + (kx - x + relX - 1)];
        }
      }
      myP[k] = s;
      mx = fmaxf(mx, s);
    }
    mx = warpMax(mx);
    float sum = 0.0f;
    for(int k = lane; k < S; k += 32) {
      const float e = (sMask[k] != 0.0f) ? expf(myP[k] - mx) : 0.0f;
      myP[k] = e;
      sum += e;
    }
    sum = warpSum(sum);
    __syncwarp();
    const float inv = 1.0f / sum;
    for(int d = lane; d < dv; d += 32) {
      float acc = 0.0f;
      for(int k = 0; k < S; k++) acc = fmaf(myP[k], sV[k * vp + d], acc);
      o[d] = fToT<T>(acc * inv);
    }
    __syncwarp();
  }
}

size_t attentionSmemBytes(int X, int Y, int dq, int dv) {
  const size_t S = (size_t)X * Y;
  return (S * (dq + 1) + S * (dv + 1) + S + 8 * S + 8 * (size_t)dq) * sizeof(float);
}
bool attentionFits(int X, int Y, int dq, int dv) { return attentionSmemBytes(X, Y, dq, dv) <= 227 * 1024; }

cudaError_t launchAttention(
  cudaStream_t st, int dt, const void* qkv, int stride, int qOff, int kOff, int vOff, int heads, int kvHeads, int dq, int dv,
  const float* mask, void* out, int outStride, Geom g, const float* relBias, int relY, int relX) {
  const size_t smem = attentionSmemBytes(g.X, g.Y, dq, dv);
  if(smem > 227 * 1024) return cudaErrorInvalidValue;
  dim3 grid((g.S + 31) / 32, g.n * heads);
  switch(dt) {
    case DT_F32: cudaFuncSetAttribute(attentionKernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); break;
    case DT_F16: cudaFuncSetAttribute(attentionKernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); break;
    default: cudaFuncSetAttribute(attentionKernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); break;
  }
  KBT_DISPATCH_DT(dt, (attentionKernel<T><<<grid, 256, smem, st>>>(
    (const T*)qkv, stride, qOff, kOff, vOff, heads, kvHeads, dq, dv, mask, (T*)out, outStride, g, relBias, relY, relX)));
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// SwiGLU

template <typename T>
__global__ void swigluKernel(const T* __restrict__ in, int inStride, T* __restrict__ out, int outStride, int C, Geom g) {
  const size_t total = (size_t)g.rowsPad * C;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / C;
    const int c = (int)(idx - m * C);
    const float a = tToF<T>(in[m * inStride + c]);
    const float b = tToF<T>(in[m * inStride + C + c]);
    out[m * outStride + c] = fToT<T>((a / (1.0f + expf(-a))) * b);
  }
}

template <typename T>
__global__ void swigluVec8Kernel(const T* __restrict__ in, int inStride, T* __restrict__ out, int outStride, int C, Geom g) {
  const int vecs = C / 8;
  const size_t total = (size_t)g.rowsPad * vecs;
  for(size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / vecs;
    const int c = (int)(idx - m * vecs) * 8;
    const uint4 av = *reinterpret_cast<const uint4*>(in + m * inStride + c);
    const uint4 bv = *reinterpret_cast<const uint4*>(in + m * inStride + C + c);
    const T* ae = reinterpret_cast<const T*>(&av);
    const T* be = reinterpret_cast<const T*>(&bv);
    uint4 ov;
    T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
    for(int j = 0; j < 8; j++) {
      const float x = tToF<T>(ae[j]);
      oe[j] = fToT<T>(__fdividef(x, 1.0f + __expf(-x)) * tToF<T>(be[j]));
    }
    *reinterpret_cast<uint4*>(out + m * outStride + c) = ov;
  }
}

cudaError_t launchSwiGLU(cudaStream_t st, int dt, const void* in, int inStride, void* out, int outStride, int C, Geom g) {
  if(dt != DT_F32 && (C % 8) == 0 && (inStride % 8) == 0 && (outStride % 8) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
     (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t totalV = (size_t)g.rowsPad * (C / 8);
    int gridV = (int)((totalV + 255) / 256);
    if(gridV > 148 * 32) gridV = 148 * 32;
    if(dt == DT_F16) swigluVec8Kernel<__half><<<gridV, 256, 0, st>>>((const __half*)in, inStride, (__half*)out, outStride, C, g);
    else swigluVec8Kernel<__nv_bfloat16><<<gridV, 256, 0, st>>>((const __nv_bfloat16*)in, inStride, (__nv_bfloat16*)out, outStride, C, g);
    return cudaGetLastError();
  }
  size_t total = (size_t)g.rowsPad * C;
  int grid = (int)((total + 255) / 256);
  if(grid > 148 * 32) grid = 148 * 32;
  KBT_DISPATCH_DT(dt, (swigluKernel<T><<<grid, 256, 0, st>>>((const T*)in, inStride, (T*)out, outStride, C, g)));
  return cudaGetLastError();
}

}  // namespace kb
