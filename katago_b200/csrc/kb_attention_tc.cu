// Attention over the points of one board on sm_100a tensor cores (tcgen05), for head dimension 64.
//
// One CTA = one (board, head); it loads K and V once and walks the board's 128-query tiles.  The tokens of a board are its padded rows (row = y*RW + x,
// kb_kernels.cuh): contiguous in memory, so Q, K and V tiles are plain 2-D TMA boxes of the QKV matrix; padding
// rows and off-board points are excluded as keys by the board mask and produce zero output as queries
// (eigenbackend.cpp:1505-1536).  All keys of a board (<= 384 rows) are processed in one pass:
//   S = Q K^T      12 MMAs 128x128x16 into 384 TMEM columns (fp32)
//   softmax        one thread per query row reads its row of S from TMEM twice (max, then exp and sum),
//                  writes P in the activation dtype into shared memory in the K-major swizzled operand layout
//   O = P V        24 MMAs 128x64x16; V is used as it lies in memory (dv contiguous = MN-major B operand)
//   out = O / sum  read from TMEM, written with 16-byte stores
// Waits are bounded as in the convolution kernel; on a time-out the status word is set and the CTA runs
// through its remaining barriers without touching data.
#include "kb_kernels.cuh"
#include "kb_tc_ptx.cuh"

#include <mutex>

namespace kb {

constexpr int AT_SK = 384;     // keys per board handled in one pass (19x19: 19*20 = 380 rows)
constexpr int AT_D = 64;       // head dimension (q, k and v)
constexpr int AT_THREADS = 256;
constexpr int AT_TILE_BYTES = 128 * 128;  // 128 rows x 64 elements x 2 bytes

enum { AT_ERR_TIMEOUT = 201 };

struct AttnTcArgs {
  Geom g;
  int heads, kvHeads;
  int qOff, kOff, vOff;   // column offsets of Q, K, V in the QKV matrix
  int keysValid;          // Y * RW: rows of a board that can hold keys
  const float* mask;
  void* out;
  int outStride;
  uint32_t idescS, idescO;
  float scaleLog2e;       // 1/sqrt(dq) * log2(e)
  int* status;
};

template <typename T> struct AtPack;
template <> struct AtPack<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
};
template <> struct AtPack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
};

// MN-major B operand (V): 64 contiguous elements (128 B) per key row, 128-byte swizzle; the K dimension (keys)
// advances by rows, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t makeSmemDescMN(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset: unused, a single 64-element MN atom
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-key groups
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <typename T>
__global__ void __launch_bounds__(AT_THREADS, 1) attentionTcKernel(const __grid_constant__ CUtensorMap tmQKV, const AttnTcArgs a) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                         // 16 KiB
  uint8_t* sK = sQ + AT_TILE_BYTES;           // 3 x 16 KiB (128 keys each)
  uint8_t* sV = sK + 3 * AT_TILE_BYTES;       // 3 x 16 KiB
  uint8_t* sP = sV + 3 * AT_TILE_BYTES;       // 6 x 16 KiB (64 keys each), K-major operand layout
  float* sMask = reinterpret_cast<float*>(sP + 6 * AT_TILE_BYTES);  // [AT_SK]
  float* sRed = sMask + AT_SK;                                      // [2][128] partial row maxima, then partial row sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRed + 256);         // kv, q, mma1, mma2
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3;        // TMEM lane quarter this warp may read
  const int half = warp >> 2;          // which half of the keys (softmax) / of the output columns this warp handles
  const int row = quarter * 32 + lane; // query row inside the tile
  const int n = blockIdx.x / a.heads, h = blockIdx.x % a.heads;
  const int kvh = h / (a.heads / a.kvHeads);
  const int boardRow = n * a.g.PB;
  const int numQTiles = (a.keysValid + 127) / 128;

  if(tid == 0) {
    for(int i = 0; i < 4; i++) mbarInit(smemU32(&bars[i]), 1);
    *abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 0) { tmemAlloc(smemU32(tmemSlot), 512); tmemRelinquish(); }
  for(int j = tid; j < AT_SK; j += AT_THREADS) sMask[j] = (j < a.keysValid) ? a.mask[boardRow + j] : 0.0f;
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const uint32_t tmemS = tmemBase, tmemO = tmemBase + AT_SK;

  if(tid == 0) {
    // K and V of this (board, kv head) are loaded once and serve every query tile; the first Q tile rides along
    mbarExpectTx(smemU32(&bars[0]), 6u * AT_TILE_BYTES);
    for(int j = 0; j < 3; j++) {
      tmaLoad2d(smemU32(sK + j * AT_TILE_BYTES), &tmQKV, a.kOff + kvh * AT_D, boardRow + j * 128, smemU32(&bars[0]));
      tmaLoad2d(smemU32(sV + j * AT_TILE_BYTES), &tmQKV, a.vOff + kvh * AT_D, boardRow + j * 128, smemU32(&bars[0]));
    }
    mbarExpectTx(smemU32(&bars[1]), (uint32_t)AT_TILE_BYTES);
    tmaLoad2d(smemU32(sQ), &tmQKV, a.qOff + h * AT_D, boardRow, smemU32(&bars[1]));
  }

  for(int qt = 0; qt < numQTiles; qt++) {
    const uint32_t ph = (uint32_t)qt & 1u;
    const int q0 = qt * 128;
    if(tid == 0) {
      bool ok = (qt > 0 || mbarWait(smemU32(&bars[0]), 0u, abortFlag)) && mbarWait(smemU32(&bars[1]), ph, abortFlag);
      if(ok) {
        tcFenceAfter();
        for(int j = 0; j < 3; j++) {
#pragma unroll
          for(int k = 0; k < AT_D / 16; k++)
            umma(tmemS + (uint32_t)(j * 128), makeSmemDesc(smemU32(sQ) + k * 32), makeSmemDesc(smemU32(sK + j * AT_TILE_BYTES) + k * 32), a.idescS, k > 0 ? 1u : 0u);
        }
        ummaCommit(smemU32(&bars[2]));
      }
      else if(!*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, AT_ERR_TIMEOUT); }
    }
    // ---- softmax: two warps per query row quarter, each over half of the keys ----
    const float qMask = (q0 + row < a.keysValid) ? a.mask[boardRow + q0 + row] : 0.0f;
    bool ok = mbarWait(smemU32(&bars[2]), ph, abortFlag);
    if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, AT_ERR_TIMEOUT); }
    if(tid == 0 && ok && qt + 1 < numQTiles) {
      // S = Q K^T has completed, so the Q tile is free: fetch the next one behind the softmax
      mbarExpectTx(smemU32(&bars[1]), (uint32_t)AT_TILE_BYTES);
      tmaLoad2d(smemU32(sQ), &tmQKV, a.qOff + h * AT_D, boardRow + q0 + 128, smemU32(&bars[1]));
    }
    const int cBegin = half * (AT_SK / 2), cEnd = cBegin + AT_SK / 2;
    float mx = -1e30f;
    if(ok) {
      tcFenceAfter();
      for(int c = cBegin; c < cEnd; c += 32) {
        uint32_t r[32];
        tmemLd32(tmemS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, r);
        tmemLdWait();
#pragma unroll
        for(int j = 0; j < 32; j++)
          if(sMask[c + j] != 0.0f) mx = fmaxf(mx, __uint_as_float(r[j]));
      }
    }
    sRed[half * 128 + row] = mx;
    __syncthreads();
    mx = fmaxf(sRed[row], sRed[128 + row]);
    __syncthreads();
    float sum = 0.0f;
    if(ok) {
      const int sw = row & 7;
      for(int c = cBegin; c < cEnd; c += 32) {
        uint32_t r[32];
        tmemLd32(tmemS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, r);
        tmemLdWait();
        float p[32];
#pragma unroll
        for(int j = 0; j < 32; j++) {
          p[j] = (sMask[c + j] != 0.0f) ? exp2f((__uint_as_float(r[j]) - mx) * a.scaleLog2e) : 0.0f;
          sum += p[j];
        }
        // P chunk of 64 keys = one 128-byte swizzled row per query; this 32-key group is its half (c/32)&1
        uint8_t* pRow = sP + (size_t)(c / 64) * AT_TILE_BYTES + row * 128;
        const int halfSel = (c / 32) & 1;
#pragma unroll
        for(int jj = 0; jj < 4; jj++) {
          uint4 o;
          o.x = AtPack<T>::pack(p[8 * jj], p[8 * jj + 1]); o.y = AtPack<T>::pack(p[8 * jj + 2], p[8 * jj + 3]);
          o.z = AtPack<T>::pack(p[8 * jj + 4], p[8 * jj + 5]); o.w = AtPack<T>::pack(p[8 * jj + 6], p[8 * jj + 7]);
          *reinterpret_cast<uint4*>(pRow + (((halfSel * 4 + jj) ^ sw) << 4)) = o;
        }
      }
    }
    sRed[half * 128 + row] = sum;
    fenceProxyAsync();
    tcFenceBefore();
    __syncthreads();
    const float rowSum = sRed[row] + sRed[128 + row];
    if(tid == 0 && !*abortFlag) {
      tcFenceAfter();
      uint32_t acc = 0;
      for(int kc = 0; kc < AT_SK / 64; kc++) {
#pragma unroll
        for(int k = 0; k < 4; k++) {
          const uint32_t pAddr = smemU32(sP + (size_t)kc * AT_TILE_BYTES) + k * 32;  // 16 keys further along K inside the atom
          const uint32_t vAddr = smemU32(sV) + (uint32_t)(kc * 64 + k * 16) * 128u;   // 16 key rows further
          umma(tmemO, makeSmemDesc(pAddr), makeSmemDescMN(vAddr), a.idescO, acc);
          acc = 1;
        }
      }
      ummaCommit(smemU32(&bars[3]));
    }
    ok = !*abortFlag && mbarWait(smemU32(&bars[3]), ph, abortFlag);
    if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, AT_ERR_TIMEOUT); }
    if(ok) {
      tcFenceAfter();
      const float inv = (qMask != 0.0f && rowSum > 0.0f) ? 1.0f / rowSum : 0.0f;
      uint32_t r[32];
      tmemLd32(tmemO + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 32), r);
      tmemLdWait();
      if(q0 + row < a.g.PB) {
        T* o = reinterpret_cast<T*>(a.out) + (size_t)(boardRow + q0 + row) * a.outStride + h * AT_D + half * 32;
#pragma unroll
        for(int jj = 0; jj < 4; jj++) {
          uint4 v;
          v.x = AtPack<T>::pack(__uint_as_float(r[8 * jj]) * inv, __uint_as_float(r[8 * jj + 1]) * inv);
          v.y = AtPack<T>::pack(__uint_as_float(r[8 * jj + 2]) * inv, __uint_as_float(r[8 * jj + 3]) * inv);
          v.z = AtPack<T>::pack(__uint_as_float(r[8 * jj + 4]) * inv, __uint_as_float(r[8 * jj + 5]) * inv);
          v.w = AtPack<T>::pack(__uint_as_float(r[8 * jj + 6]) * inv, __uint_as_float(r[8 * jj + 7]) * inv);
          *reinterpret_cast<uint4*>(o + 8 * jj) = v;
        }
      }
    }
    // every warp has finished reading S and O of this tile before the next tile's MMAs overwrite them
    tcFenceBefore();
    __syncthreads();
    tcFenceAfter();
  }
  if(warp == 0) { tcFenceAfter(); tmemDealloc(tmemBase, 512); }
}

// ---------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFnA)(
  CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct AttnTcPlan {
  CUtensorMap tmQKV;
  int dt;
  size_t smemBytes;
};

bool attentionTcEligible(int dt, int dq, int dv, int X, int Y, int stride, int qOff, int kOff, int vOff, int outStride) {
  if(dt != DT_F16 && dt != DT_BF16) return false;
  if(dq != AT_D || dv != AT_D) return false;
  if(Y * (X + 1) > AT_SK) return false;
  if((stride % 8) || (qOff % 8) || (kOff % 8) || (vOff % 8) || (outStride % 8)) return false;
  return true;
}

AttnTcPlan* attentionTcCreate(int dt, const void* qkv, int stride, int totalCols, int rowsPadMax) {
  static EncodeTiledFnA fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnA>(p);
  });
  if(!fn || (reinterpret_cast<uintptr_t>(qkv) & 15)) return nullptr;
  AttnTcPlan* p = new AttnTcPlan();
  p->dt = dt;
  cuuint64_t dims[2] = {(cuuint64_t)totalCols, (cuuint64_t)rowsPadMax};
  cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
  cuuint32_t box[2] = {AT_D, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(
    &p->tmQKV, dt == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides,
    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if(r != CUDA_SUCCESS) { delete p; return nullptr; }
  p->smemBytes = 13 * (size_t)AT_TILE_BYTES + (AT_SK + 256) * sizeof(float) + 4 * 8 + 16 + 1024;
  cudaError_t e1 = cudaFuncSetAttribute(attentionTcKernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smemBytes);
  cudaError_t e2 = cudaFuncSetAttribute(attentionTcKernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smemBytes);
  if(e1 != cudaSuccess || e2 != cudaSuccess) { delete p; return nullptr; }
  return p;
}

void attentionTcDestroy(AttnTcPlan* p) { delete p; }

cudaError_t launchAttentionTc(
  cudaStream_t st, const AttnTcPlan* p, int qOff, int kOff, int vOff, int heads, int kvHeads, const float* mask, void* out,
  int outStride, Geom g, int* statusWord) {
  AttnTcArgs a;
  a.g = g; a.heads = heads; a.kvHeads = kvHeads; a.qOff = qOff; a.kOff = kOff; a.vOff = vOff;
  a.keysValid = g.Y * g.RW;
  a.mask = mask; a.out = out; a.outStride = outStride;
  const uint32_t fmt = p->dt == DT_F16 ? 0u : 1u;
  a.idescS = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.idescO = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(AT_D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.scaleLog2e = 1.4426950408889634f / sqrtf((float)AT_D);
  a.status = statusWord;
  dim3 grid(g.n * heads);
  if(p->dt == DT_F16) attentionTcKernel<__half><<<grid, AT_THREADS, p->smemBytes, st>>>(p->tmQKV, a);
  else attentionTcKernel<__nv_bfloat16><<<grid, AT_THREADS, p->smemBytes, st>>>(p->tmQKV, a);
  return cudaGetLastError();
}

}  // namespace kb
