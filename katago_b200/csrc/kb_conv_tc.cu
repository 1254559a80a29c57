// Tensor-core convolution for sm_100a: 1x1 and 3x3 convolutions as implicit GEMM on tcgen05
// with the accumulators in tensor memory (TMEM), operands staged into shared memory by TMA,
// and the next layer's norm + activation + mask (and the residual add) fused into the epilogue.
//
// GEMM view.  D[row][oc] = sum over taps t and input channels ic of A[row + shift(t)][ic] * W[t][oc][ic],
// where rows are the padded-rows layout of kb_kernels.cuh: because every board line and every
// board carry one line/column of zeros, shift(t) = dy*RW + dx is a constant row offset.
//
// A operand ("halo tile").  For one tile of 128 output rows and one chunk of 64 input channels, ONE TMA
// box of 128 + 2*halo rows is loaded (rows before the tensor start or past its end are zero-filled by
// TMA).  The nine taps of a 3x3 convolution read the same shared-memory tile through nine shared-memory
// matrix descriptors whose start address is moved by shift(t) rows; activations therefore cross the
// L2 -> SM path once per tile instead of nine times.  The weight tile of each (tap, chunk) streams
// through a ring of slots.
//
// Persistent CTAs (one per SM), 320 threads: warp 0 issues TMA loads, warp 1 owns TMEM and issues the
// MMAs, warps 2..9 run the epilogue (two warps per TMEM lane quarter, alternating 16-column groups).
// Two accumulators live in TMEM, so the epilogue of tile i overlaps the main loop of tile i+1.
// Every wait is bounded: on time-out the kernel records a code in the status word and all roles
// leave through the common exit, which still frees TMEM.
#include "kb_kernels.cuh"
#include "../../include/kb_modelblob.h"

#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace kb {

// ---------------------------------------------------------------------------------------------
// PTX wrappers

__device__ __forceinline__ uint32_t smemU32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbarTryWait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(ok)
    : "r"(bar), "r"(parity)
    : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait (about 2 s).  Returns false on time-out or if another role already gave up.
__device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity, volatile int* abortFlag) {
  if(mbarTryWait(bar, parity)) return true;
  const uint64_t t0 = globalTimerNs();
  uint32_t spins = 0;
  while(true) {
    if(mbarTryWait(bar, parity)) return true;
    if((++spins & 63u) == 0u) {
      if(*abortFlag) return false;
      if(globalTimerNs() - t0 > 2000000000ull) return false;
    }
  }
}

__device__ __forceinline__ void tmaLoad2d(uint32_t dst, const CUtensorMap* tmap, int c0, int c1, uint32_t bar) {
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
    ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
    : "memory");
}

__device__ __forceinline__ void tmemAlloc(uint32_t dstSmem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], M=128, N from idesc, K=16 (fp16/bf16), fp32 accumulate.
__device__ __forceinline__ void umma(uint32_t dTmem, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
    ::"r"(dTmem), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
    : "memory");
}
// mbarrier arrives once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void ummaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread t reads lane base+t).
__device__ __forceinline__ void tmemLd32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
    : "r"(taddr)
    : "memory");
}
__device__ __forceinline__ void tmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 B apart, 8-row groups
// 1024 B apart (stride byte offset), descriptor version 1 (Blackwell).  The swizzle is a function of the
// absolute shared-memory address bits, so a start address moved by whole rows (any multiple of 128 B) or by
// 32-byte K steps inside the atom addresses the data exactly where TMA put it; the base-offset field stays 0
// (measured: results match the CUDA-core kernel bit for bit in that configuration only).
__device__ __forceinline__ uint64_t makeSmemDesc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
  d |= (uint64_t)1 << 46;                    // version
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}

// ---------------------------------------------------------------------------------------------
// Fast activations for the reduced-precision epilogue

__device__ __forceinline__ float fastMish(float x) {
  // x*tanh(softplus(x)) = x * w/(w+2), w = e^x (e^x + 2); exact identity, evaluated with ex2/rcp approximations.
  float e = __expf(fminf(x, 20.0f));
  float w = e * (e + 2.0f);
  return x * __fdividef(w, w + 2.0f);
}
__device__ __forceinline__ float fastAct(float x, int act) {
  switch(act) {
    case KB_ACT_RELU: return fmaxf(x, 0.0f);
    case KB_ACT_MISH: return fastMish(x);
    case KB_ACT_SILU: return __fdividef(x, 1.0f + __expf(-x));
    case KB_ACT_MISH_SCALE8: {
      float e = __expf(fminf(8.0f * x, 20.0f));
      float w = e * (e + 2.0f);
      return x * __fdividef(w, w + 2.0f);
    }
    default: return x;
  }
}

template <typename T> struct Pack2;
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
};
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
};


// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread (thread t reads lane base+t).
__device__ __forceinline__ void tmemLd16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
    : "r"(taddr)
    : "memory");
}

// ---------------------------------------------------------------------------------------------
// Kernel

struct ConvTcArgs {
  Geom g;
  Epilogue ep;
  int inC, outC, kY, kX;
  int BN;          // output channels per tile (multiple of 16, <= 256)
  int kChunks;     // inC / 64
  int haloPad;     // rows loaded above the tile (multiple of 8, >= largest upward shift); 0 for 1x1
  int aRows;       // rows of the A halo tile (TMA box height)
  int aSlotBytes;  // aRows * 128
  int bSlotBytes;  // BN * 128
  int numA, numB;  // ring depths
  uint32_t idesc;
  uint32_t tmemCols;
  int* status;     // device status word: 0 = ok
};

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_THREADS = 320;
constexpr int TC_EPI_WARPS = 8;

enum { TC_ERR_PRODUCER_TIMEOUT = 101, TC_ERR_MMA_TIMEOUT = 102, TC_ERR_EPILOGUE_TIMEOUT = 103 };

// One group of 16 output channels of one row: bias, residual, raw store, norm+activation store.
template <typename T, int ACT>
__device__ __forceinline__ void epilogue16(
  const uint32_t (&r)[16], const Epilogue& ep, int m, int c, float mk, const float* biasRow, const float* sScale, const float* sBias) {
  float v[16];
#pragma unroll
  for(int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
  if(biasRow) {
    const float4* bp = reinterpret_cast<const float4*>(biasRow + c);
#pragma unroll
    for(int j = 0; j < 4; j++) {
      float4 b4 = bp[j];
      v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
    }
  }
  if(ep.residual) {
    const uint4* rp = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(ep.residual) + (size_t)m * ep.resStride + c);
    uint4 r0 = rp[0], r1 = rp[1];
    const uint32_t ru[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
    for(int j = 0; j < 8; j++) {
      float2 f = Pack2<T>::unpack(ru[j]);
      v[2 * j] += f.x;
      v[2 * j + 1] += f.y;
    }
  }
  if(ep.outRaw && c >= ep.rawC0 && c < ep.rawC1) {
    uint32_t pk[8];
#pragma unroll
    for(int j = 0; j < 8; j++) pk[j] = Pack2<T>::pack(v[2 * j], v[2 * j + 1]);
    uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<T*>(ep.outRaw) + (size_t)m * ep.rawStride + (c - ep.rawC0));
    op[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    op[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  }
  if(ep.outAct && c >= ep.actC0 && c < ep.actC1) {
    const int ca = c - ep.actC0;
    uint32_t pk[8];
    if(mk == 1.0f) {
      const float4* sp = reinterpret_cast<const float4*>(sScale + ca);
      const float4* bp = reinterpret_cast<const float4*>(sBias + ca);
      float o[16];
#pragma unroll
      for(int j = 0; j < 4; j++) {
        const float4 s4 = sp[j], b4 = bp[j];
        o[4 * j] = fastAct(fmaf(v[4 * j], s4.x, b4.x), ACT);
        o[4 * j + 1] = fastAct(fmaf(v[4 * j + 1], s4.y, b4.y), ACT);
        o[4 * j + 2] = fastAct(fmaf(v[4 * j + 2], s4.z, b4.z), ACT);
        o[4 * j + 3] = fastAct(fmaf(v[4 * j + 3], s4.w, b4.w), ACT);
      }
#pragma unroll
      for(int j = 0; j < 8; j++) pk[j] = Pack2<T>::pack(o[2 * j], o[2 * j + 1]);
    }
    else {
#pragma unroll
      for(int j = 0; j < 8; j++) pk[j] = 0u;
    }
    uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<T*>(ep.outAct) + (size_t)m * ep.actStride + ca);
    op[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    op[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  }
}

// All 16-column groups of one tile that belong to this warp (groups alternate between the two warps of a quarter).
template <typename T, int ACT>
__device__ __forceinline__ void epilogueTile(
  const ConvTcArgs& a, uint32_t tmemAcc, int q, int half, int m, int n0, const float* sScale, const float* sBias) {
  const Epilogue& ep = a.ep;
  const float mk = ep.mask ? ep.mask[m] : 1.0f;
  const int b = min(m / a.g.PB, a.g.n - 1);
  const float* biasRow = ep.biasNC ? ep.biasNC + (size_t)b * a.outC : nullptr;
  const int groups = a.BN / 16;
  for(int gi = half; gi < groups; gi += 2) {
    uint32_t r[16];
    tmemLd16(tmemAcc + ((uint32_t)(q * 32) << 16) + (uint32_t)(gi * 16), r);
    tmemLdWait();
    epilogue16<T, ACT>(r, ep, m, n0 + gi * 16, mk, biasRow, sScale, sBias);
  }
}

template <typename T>
__global__ void __launch_bounds__(TC_THREADS, 1) convTcKernel(
  const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const ConvTcArgs a) {
  extern __shared__ uint8_t smemRaw[];
  // 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smemA + (size_t)a.numA * a.aSlotBytes;
  float* sScale = reinterpret_cast<float*>(smemB + (size_t)a.numB * a.bSlotBytes);
  float* sBias = sScale + 512;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sBias + 512);
  // barrier layout: fullA[numA] emptyA[numA] fullB[numB] emptyB[numB] accFull[2] accEmpty[2]
  uint64_t* fullA = bars;
  uint64_t* emptyA = fullA + a.numA;
  uint64_t* fullB = emptyA + a.numA;
  uint64_t* emptyB = fullB + a.numB;
  uint64_t* accFull = emptyB + a.numB;
  uint64_t* accEmpty = accFull + 2;
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmpty + 2);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int numNTiles = a.outC / a.BN;
  const int numTiles = (a.g.rowsPad / TC_BM) * numNTiles;
  const int taps = a.kY * a.kX;

  if(threadIdx.x == 0) {
    for(int s = 0; s < a.numA; s++) { mbarInit(smemU32(&fullA[s]), 1); mbarInit(smemU32(&emptyA[s]), 1); }
    for(int s = 0; s < a.numB; s++) { mbarInit(smemU32(&fullB[s]), 1); mbarInit(smemU32(&emptyB[s]), 1); }
    for(int s = 0; s < 2; s++) { mbarInit(smemU32(&accFull[s]), 1); mbarInit(smemU32(&accEmpty[s]), TC_EPI_WARPS); }
    *abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 1) {
    tmemAlloc(smemU32(tmemSlot), a.tmemCols);
    tmemRelinquish();
  }
  // next layer's norm parameters: read once per CTA
  if(a.ep.outAct) {
    const int nAct = a.ep.actC1 - a.ep.actC0;
    for(int i = threadIdx.x; i < nAct; i += blockDim.x) { sScale[i] = a.ep.scale[i]; sBias[i] = a.ep.bias[i]; }
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  if(warp == 0) {
    // ---------------- TMA producer ----------------
    if(lane == 0) {
      uint32_t ia = 0, ib = 0;
      bool ok = true;
      for(int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        const int m0 = (t / numNTiles) * TC_BM, n0 = (t % numNTiles) * a.BN;
        for(int kc = 0; kc < a.kChunks && ok; kc++) {
          const uint32_t sa = ia % a.numA;
          if(!mbarWait(smemU32(&emptyA[sa]), ((ia / a.numA) & 1u) ^ 1u, abortFlag)) { ok = false; break; }
          mbarExpectTx(smemU32(&fullA[sa]), (uint32_t)a.aSlotBytes);
          tmaLoad2d(smemU32(smemA + (size_t)sa * a.aSlotBytes), &tmA, kc * TC_BK, m0 - a.haloPad, smemU32(&fullA[sa]));
          ia++;
          for(int tap = 0; tap < taps; tap++) {
            const uint32_t sb = ib % a.numB;
            if(!mbarWait(smemU32(&emptyB[sb]), ((ib / a.numB) & 1u) ^ 1u, abortFlag)) { ok = false; break; }
            mbarExpectTx(smemU32(&fullB[sb]), (uint32_t)a.bSlotBytes);
            tmaLoad2d(smemU32(smemB + (size_t)sb * a.bSlotBytes), &tmB, kc * TC_BK, tap * a.outC + n0, smemU32(&fullB[sb]));
            ib++;
          }
        }
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_PRODUCER_TIMEOUT); }
    }
  }
  else if(warp == 1) {
    // ---------------- MMA issuer ----------------
    if(lane == 0) {
      uint32_t ia = 0, ib = 0, it = 0;
      bool ok = true;
      for(int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, it++) {
        const uint32_t buf = it & 1u;
        // wait until the epilogue has drained this accumulator (two tiles ago)
        if(!mbarWait(smemU32(&accEmpty[buf]), ((it >> 1) & 1u) ^ 1u, abortFlag)) { ok = false; break; }
        tcFenceAfter();
        const uint32_t dTmem = tmemBase + buf * (uint32_t)a.BN;
        uint32_t first = 1;
        for(int kc = 0; kc < a.kChunks && ok; kc++) {
          const uint32_t sa = ia % a.numA;
          if(!mbarWait(smemU32(&fullA[sa]), (ia / a.numA) & 1u, abortFlag)) { ok = false; break; }
          const uint32_t aBase = smemU32(smemA + (size_t)sa * a.aSlotBytes);
          for(int tap = 0; tap < taps; tap++) {
            const uint32_t sb = ib % a.numB;
            if(!mbarWait(smemU32(&fullB[sb]), (ib / a.numB) & 1u, abortFlag)) { ok = false; break; }
            tcFenceAfter();
            const int dy = tap / a.kX - a.kY / 2, dx = tap % a.kX - a.kX / 2;
            const uint32_t aStart = aBase + (uint32_t)(a.haloPad + dy * a.g.RW + dx) * 128u;
            const uint32_t bStart = smemU32(smemB + (size_t)sb * a.bSlotBytes);
#pragma unroll
            for(int k = 0; k < TC_BK / 16; k++) {
              // advancing K by 16 elements = 32 bytes inside the 128-byte swizzle atom
              umma(dTmem, makeSmemDesc(aStart + k * 32), makeSmemDesc(bStart + k * 32), a.idesc, first ? 0u : 1u);
              first = 0;
            }
            ummaCommit(smemU32(&emptyB[sb]));  // frees the weight slot once these MMAs have read it
            ib++;
          }
          ummaCommit(smemU32(&emptyA[sa]));
          ia++;
        }
        if(ok) ummaCommit(smemU32(&accFull[buf]));
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_MMA_TIMEOUT); }
    }
  }
  else {
    // ---------------- Epilogue: warps 2..9; TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t it = 0;
    for(int t = blockIdx.x; t < numTiles; t += gridDim.x, it++) {
      const uint32_t buf = it & 1u;
      const int m0 = (t / numNTiles) * TC_BM, n0 = (t % numNTiles) * a.BN;
      bool ok = mbarWait(smemU32(&accFull[buf]), (it >> 1) & 1u, abortFlag);
      ok = __all_sync(0xffffffffu, ok);
      if(!ok) {
        if(lane == 0 && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_EPILOGUE_TIMEOUT); }
        break;
      }
      tcFenceAfter();
      const uint32_t acc = tmemBase + buf * (uint32_t)a.BN;
      const int m = m0 + q * 32 + lane;
      switch(a.ep.act) {
        case KB_ACT_RELU: epilogueTile<T, KB_ACT_RELU>(a, acc, q, half, m, n0, sScale, sBias); break;
        case KB_ACT_MISH: epilogueTile<T, KB_ACT_MISH>(a, acc, q, half, m, n0, sScale, sBias); break;
        case KB_ACT_SILU: epilogueTile<T, KB_ACT_SILU>(a, acc, q, half, m, n0, sScale, sBias); break;
        case KB_ACT_MISH_SCALE8: epilogueTile<T, KB_ACT_MISH_SCALE8>(a, acc, q, half, m, n0, sScale, sBias); break;
        default: epilogueTile<T, KB_ACT_IDENTITY>(a, acc, q, half, m, n0, sScale, sBias); break;
      }
      // all TMEM reads of this warp are complete (tcgen05.wait::ld inside): hand the accumulator back
      tcFenceBefore();
      __syncwarp();
      if(lane == 0) mbarArrive(smemU32(&accEmpty[buf]));
    }
  }

  // ---------------- common exit ----------------
  tcFenceBefore();
  __syncthreads();
  if(*abortFlag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before the shared memory is released
    const uint64_t t0 = globalTimerNs();
    while(globalTimerNs() - t0 < 2000000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  if(warp == 1) {
    tcFenceAfter();
    tmemDealloc(tmemBase, a.tmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side

typedef CUresult (*EncodeTiledFn)(
  CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn getEncodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
       qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct ConvTcPlan {
  CUtensorMap tmA, tmB;
  int dt, inC, outC, kY, kX, X, Y;
  int BN, kChunks, haloPad, aRows, aSlotBytes, bSlotBytes, numA, numB;
  uint32_t idesc, tmemCols;
  size_t smemBytes;
  int numSMs;
};

static int pickBN(int outC) {
  // largest multiple of 16 that divides outC and fits one MMA (N <= 256)
  for(int bn = 256; bn >= 16; bn -= 16)
    if(outC % bn == 0) return bn;
  return 0;
}

bool convTcEligible(int dt, int inC, int outC, int kY, int kX) {
  if(dt != DT_F16 && dt != DT_BF16) return false;
  if(!((kY == 1 && kX == 1) || (kY == 3 && kX == 3))) return false;
  if(inC % TC_BK != 0 || outC % 16 != 0 || outC > 512) return false;
  return pickBN(outC) >= 16;
}

static bool encode2d(CUtensorMap* tm, int dt, const void* base, uint64_t inner, uint64_t outer, uint64_t strideBytes, uint32_t boxInner, uint32_t boxOuter) {
  EncodeTiledFn fn = getEncodeTiled();
  if(!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {strideBytes};
  cuuint32_t box[2] = {boxInner, boxOuter};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(
    tm, dt == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

ConvTcPlan* convTcCreate(
  int dt, const void* in, int inStride, int inC, const void* w, int outC, int kY, int kX, int X, int Y, int rowsPadMax) {
  if(!convTcEligible(dt, inC, outC, kY, kX)) return nullptr;
  if((inStride % 8) != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return nullptr;
  ConvTcPlan* p = new ConvTcPlan();
  p->dt = dt; p->inC = inC; p->outC = outC; p->kY = kY; p->kX = kX; p->X = X; p->Y = Y;
  p->BN = pickBN(outC);
  p->kChunks = inC / TC_BK;
  const int maxShift = (kY == 3) ? (X + 1) + 1 : 0;  // RW + 1 rows up or down
  p->haloPad = (maxShift + 7) / 8 * 8;
  p->aRows = (p->haloPad + TC_BM + maxShift + 7) / 8 * 8;
  if(p->aRows > 256) { delete p; return nullptr; }
  p->aSlotBytes = p->aRows * 128;
  p->bSlotBytes = p->BN * 128;
  p->numA = 2;
  const int fixedBytes = 2 * 512 * 4 + 64 * 8 + 64 + 1024;
  int numB = (225 * 1024 - fixedBytes - p->numA * p->aSlotBytes) / p->bSlotBytes;
  if(const char* e = getenv("KB_TC_NUMB")) { int v = atoi(e); if(v >= 1 && v <= 16) numB = v < numB ? v : numB; }
  if(numB > 12) numB = 12;
  if(numB < 2) { delete p; return nullptr; }
  p->numB = numB;
  p->smemBytes = (size_t)p->numA * p->aSlotBytes + (size_t)p->numB * p->bSlotBytes + fixedBytes;
  p->tmemCols = 32;
  while((int)p->tmemCols < 2 * p->BN) p->tmemCols *= 2;
  const uint32_t fmt = dt == DT_F16 ? 0u : 1u;
  // instruction descriptor: D=f32, A/B format, both K-major, N>>3 at bit 17, M>>4 at bit 24
  p->idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p->BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
  bool ok = encode2d(&p->tmA, dt, in, (uint64_t)inC, (uint64_t)rowsPadMax, (uint64_t)inStride * 2, TC_BK, (uint32_t)p->aRows) &&
            encode2d(&p->tmB, dt, w, (uint64_t)inC, (uint64_t)kY * kX * outC, (uint64_t)inC * 2, TC_BK, (uint32_t)p->BN);
  if(!ok) { delete p; return nullptr; }
  cudaError_t e1 = cudaFuncSetAttribute(convTcKernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  cudaError_t e2 = cudaFuncSetAttribute(convTcKernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  int dev = 0, sms = 148;
  if(cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  p->numSMs = sms;
  if(e1 != cudaSuccess || e2 != cudaSuccess) { delete p; return nullptr; }
  return p;
}

void convTcDestroy(ConvTcPlan* p) { delete p; }

cudaError_t launchConvTc(cudaStream_t st, const ConvTcPlan* p, Geom g, const Epilogue& ep, int* statusWord) {
  // vector accesses in the epilogue need 16-byte aligned rows and 16-channel aligned ranges
  if(ep.outRaw && ((ep.rawStride % 8) || (ep.rawC0 % 16) || (ep.rawC1 % 16))) return cudaErrorInvalidValue;
  if(ep.outAct && ((ep.actStride % 8) || (ep.actC0 % 16) || (ep.actC1 % 16) || (ep.actC1 - ep.actC0) > 512)) return cudaErrorInvalidValue;
  if(ep.residual && (ep.resStride % 8)) return cudaErrorInvalidValue;
  ConvTcArgs a;
  a.g = g; a.ep = ep;
  a.inC = p->inC; a.outC = p->outC; a.kY = p->kY; a.kX = p->kX;
  a.BN = p->BN; a.kChunks = p->kChunks; a.haloPad = p->haloPad; a.aRows = p->aRows;
  a.aSlotBytes = p->aSlotBytes; a.bSlotBytes = p->bSlotBytes; a.numA = p->numA; a.numB = p->numB;
  a.idesc = p->idesc; a.tmemCols = p->tmemCols;
  a.status = statusWord;
  const int numTiles = (g.rowsPad / TC_BM) * (p->outC / p->BN);
  const int grid = numTiles < p->numSMs ? numTiles : p->numSMs;
  if(p->dt == DT_F16)
    convTcKernel<__half><<<grid, TC_THREADS, p->smemBytes, st>>>(p->tmA, p->tmB, a);
  else
    convTcKernel<__nv_bfloat16><<<grid, TC_THREADS, p->smemBytes, st>>>(p->tmA, p->tmB, a);
  return cudaGetLastError();
}

}  // namespace kb
