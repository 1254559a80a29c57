// The 1x1 convolution that closes a nested bottleneck block and the 1x1 convolution that opens the next one, as one
// kernel (eigenbackend.cpp:1254-1303: trunk += postConv(act(postBN(mid))); nextMid = preConv(act(preBN(trunk)))).
//
// As two launches the pair is bound by memory: the first writes the activated trunk tensor (the widest tensor of the
// net) only for the second to read it back once.  Here the activated values never leave the SM: the epilogue of the
// first GEMM writes them, in the tensor cores' operand layout, into shared memory, from where the second GEMM takes
// its A operand.  Per 128 rows the kernel reads the block's mid tensor and the residual stream and writes the stream,
// the next block's mid stream and its activated form: 7/12 of the bytes of the two separate kernels.
//
// One persistent CTA per SM; warp 0 issues TMA loads, warp 1 issues the MMAs, warps 2..13 are epilogue warps (three per
// TMEM lane quarter).  GEMM1 (rows x Cm -> Ct) runs in parts of 128 output channels whose accumulators alternate
// between two TMEM buffers; the epilogue of a part adds the residual, stores the updated stream (TMA), and writes
// act(norm(.)) * mask into the shared-memory operand buffer; GEMM2 (rows x Ct -> Cn) consumes that buffer part by part
// (two 64-channel K chunks per part) into a third accumulator, whose epilogue stores the next mid stream and its
// activated form.  Weights of both GEMMs stream through one ring of slots.  Every wait is bounded.
#include "kb_conv_dev.cuh"

#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>
#include <algorithm>
#include <utility>

namespace kb {

#ifndef KB_PP_CG
#define KB_PP_CG 3
#endif
constexpr int PP_BM = 128;          // rows per tile
constexpr int PP_CG = KB_PP_CG;            // epilogue warps per TMEM lane quarter
constexpr int PP_EPI_WARPS = 4 * PP_CG;
constexpr int PP_THREADS = 64 + 32 * PP_EPI_WARPS;
constexpr int PP_UNIT = 32 * 64;    // staging unit: 32 rows x 32 channels of the storage type (64-byte swizzle)
constexpr int PP_CHUNK = PP_BM * 128;  // one 64-channel K chunk of an A operand: 128 rows x 128 bytes
constexpr int PP_FIXED = 512;       // barriers and the TMEM slot

// Optional timeline (build with -DKB_TC_TRACE): CTA 0 records SM cycle counts of its MMA warp and of its first epilogue
// warp for the first tiles; read back with kb_debug_trace_pp.
#ifdef KB_TC_TRACE
__device__ long long g_ppTrace[1024];
#define PPT(cond, slot) do { if(blockIdx.x == 0 && (cond) && (slot) < 1024) g_ppTrace[(slot)] = clock64(); } while(0)
#else
#define PPT(cond, slot) do { } while(0)
#endif

enum { PP_ERR_PRODUCER = 111, PP_ERR_MMA = 112, PP_ERR_EPILOGUE = 113, PP_ERR_ALIGNMENT = 114 };

struct PostPreArgs {
  Geom g;
  int Cm, Ct, Cn;          // GEMM1: Cm -> Ct (+ residual); GEMM2: Ct -> Cn
  int NP;                  // output channels of GEMM1 per part (a multiple of 96: whole K chunks, units divisible by 3)
  int parts;               // Ct / NP
  int kc1;                 // Cm / 64
  int numB1, numB2;        // slots of the two weight rings (GEMM1, GEMM2)
  int b1Slot, b2Slot;      // bytes per slot
  uint32_t idesc1, idesc2, tmemCols;
  const float* scale1; const float* bias1;   // norm + activation between the two convolutions (Ct channels)
  const float* scale2; const float* bias2;   // norm + activation after the second one (Cn channels)
  const float* mask;
  int* status;
};

// Schedule of one tile (128 rows), parts p = 0 .. parts-1 of GEMM1, K chunks c of GEMM2 (NP / 64 per part):
//   MMA warp:  G1(0) | for p: { G2(p, c0) | G1(p+1) | G2(p, c1..) } | G1(0) of the CTA's next tile
//   epilogue:  for p: e1(p) (residual add, stream store, activation -> operand chunks) | e2 (outputs of GEMM2)
// GEMM1 has ONE accumulator: its next part is issued as soon as every epilogue warp has loaded its last unit of the
// current part from TMEM, which is early in that unit, so the MMAs finish long before the epilogue gets to them.  The
// operand buffer of GEMM2 holds two K chunks that the epilogue fills and the MMA warp drains in turn.
// The weights of both GEMMs stream through one ring of slots in the order the MMA warp consumes them (a ring per GEMM
// can be configured for experiments: a slot of GEMM2 is held until the epilogue has produced its operand chunk).
// shared memory: [A1: kc1 chunks][A2: 2 chunks][weight ring(s)][staging: 3 units per epilogue warp][barriers]
template <typename T, int ACT>
__global__ void __launch_bounds__(PP_THREADS, 1) convPostPreKernel(
  const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmW2,
  const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmRaw2, const __grid_constant__ CUtensorMap tmAct2,
  const PostPreArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sA1 = smem;
  uint8_t* sA2 = sA1 + (size_t)a.kc1 * PP_CHUNK;
  uint8_t* sB1 = sA2 + 2 * PP_CHUNK;
  uint8_t* sB2 = sB1 + (size_t)a.numB1 * a.b1Slot;
  uint8_t* sStage = sB2 + (size_t)a.numB2 * a.b2Slot;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + (size_t)PP_EPI_WARPS * 3 * PP_UNIT);
  uint64_t* a1Full = bars;            // 1
  uint64_t* a1Empty = a1Full + 1;     // 1
  uint64_t* b1Full = a1Empty + 1;        // [numB1]
  uint64_t* b1Empty = b1Full + a.numB1;  // [numB1]
  uint64_t* b2Full = b1Empty + a.numB1;  // [numB2]
  uint64_t* b2Empty = b2Full + a.numB2;  // [numB2]
  uint64_t* d1Full = b2Empty + a.numB2;  // 1
  uint64_t* d1Empty = d1Full + 1;     // 1
  uint64_t* a2Full = d1Empty + 1;     // [2]
  uint64_t* a2Empty = a2Full + 2;     // [2]
  uint64_t* d2Full = a2Empty + 2;     // 1
  uint64_t* d2Empty = d2Full + 1;     // 1
  uint64_t* resFull = d2Empty + 1;    // [PP_EPI_WARPS][2]
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(resFull + PP_EPI_WARPS * 2);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int numTiles = a.g.rowsPad / PP_BM;
  const int grid = (int)gridDim.x;
  const int cpp = a.NP / 64;   // K chunks of GEMM2 per part
  const int UP = a.NP / 32;    // 32-channel units per part

  gridDepLaunch();
  if(threadIdx.x == 0) {
    mbarInit(smemU32(a1Full), 1); mbarInit(smemU32(a1Empty), 1);
    for(int s = 0; s < a.numB1; s++) { mbarInit(smemU32(&b1Full[s]), 1); mbarInit(smemU32(&b1Empty[s]), 1); }
    for(int s = 0; s < a.numB2; s++) { mbarInit(smemU32(&b2Full[s]), 1); mbarInit(smemU32(&b2Empty[s]), 1); }
    mbarInit(smemU32(d1Full), 1); mbarInit(smemU32(d1Empty), PP_EPI_WARPS);
    for(int s = 0; s < 2; s++) { mbarInit(smemU32(&a2Full[s]), 8); mbarInit(smemU32(&a2Empty[s]), 1); }  // a chunk = 2 units x 4 quarters
    mbarInit(smemU32(d2Full), 1); mbarInit(smemU32(d2Empty), PP_EPI_WARPS);
    for(int s = 0; s < PP_EPI_WARPS * 2; s++) mbarInit(smemU32(&resFull[s]), 1);
    // the swizzled operand layouts assume a 1024-byte aligned base
    *abortFlag = (smemU32(smem) & 1023u) ? 1 : 0;
    if(*abortFlag) atomicCAS(a.status, 0, PP_ERR_ALIGNMENT);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 1) { tmemAlloc(smemU32(tmemSlot), a.tmemCols); tmemRelinquish(); }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const uint32_t d1Col = 0u, d2Col = (uint32_t)a.NP;
  const bool bad = *abortFlag != 0;

  if(bad) {
    // misaligned shared memory: nothing runs
  }
  else if(warp == 0) {
    // ---------------- TMA producer ----------------
    if(lane == 0) {
      uint32_t s1 = 0, ph1 = 0, s2 = 0, ph2 = 0;
      bool ok = true;
      auto loadW1c = [&](int kc, int row, uint32_t bytes) {
        if(!ok) return;
        if(!mbarWait(smemU32(&b1Empty[s1]), ph1 ^ 1u, abortFlag)) { ok = false; return; }
        const uint32_t bar = smemU32(&b1Full[s1]);
        mbarExpectTx(bar, bytes);
        tmaLoad2d(smemU32(sB1 + (size_t)s1 * a.b1Slot), &tmW1, kc * 64, row, bar);
        if(++s1 == (uint32_t)a.numB1) { s1 = 0; ph1 ^= 1u; }
      };
      auto loadW2c = [&](int kc, uint32_t bytes) {
        if(!ok) return;
        if(a.numB2 == 0) {
          // one ring for both GEMMs: the slots are taken in the order the MMA warp consumes them
          if(!mbarWait(smemU32(&b1Empty[s1]), ph1 ^ 1u, abortFlag)) { ok = false; return; }
          const uint32_t bar = smemU32(&b1Full[s1]);
          mbarExpectTx(bar, bytes);
          tmaLoad2d(smemU32(sB1 + (size_t)s1 * a.b1Slot), &tmW2, kc * 64, 0, bar);
          if(++s1 == (uint32_t)a.numB1) { s1 = 0; ph1 ^= 1u; }
          return;
        }
        if(!mbarWait(smemU32(&b2Empty[s2]), ph2 ^ 1u, abortFlag)) { ok = false; return; }
        const uint32_t bar = smemU32(&b2Full[s2]);
        mbarExpectTx(bar, bytes);
        tmaLoad2d(smemU32(sB2 + (size_t)s2 * a.b2Slot), &tmW2, kc * 64, 0, bar);
        if(++s2 == (uint32_t)a.numB2) { s2 = 0; ph2 ^= 1u; }
      };
      const uint32_t w1Bytes = (uint32_t)a.NP * 128u, w2Bytes = (uint32_t)a.Cn * 128u;
      uint32_t it = 0;
      auto loadA1 = [&](int t) {
        // the buffer is free once the last part of the tile before has been multiplied
        if(!ok) return;
        if(!mbarWait(smemU32(a1Empty), (it & 1u) ^ 1u, abortFlag)) { ok = false; return; }
        mbarExpectTx(smemU32(a1Full), (uint32_t)(a.kc1 * PP_CHUNK));
        for(int kc = 0; kc < a.kc1; kc++) tmaLoad2d(smemU32(sA1 + (size_t)kc * PP_CHUNK), &tmA1, kc * 64, t * PP_BM, smemU32(a1Full));
        it++;
      };
      auto loadW1 = [&](int p) { for(int kc = 0; kc < a.kc1; kc++) loadW1c(kc, p * a.NP, w1Bytes); };
      gridDepWait();
      int t = (int)blockIdx.x;
      if(t < numTiles) { loadA1(t); loadW1(0); }
      for(; t < numTiles && ok; t += grid) {
        for(int p = 0; p < a.parts && ok; p++) {
          // the two rings are independent, but one thread issues both: the order follows the MMA warp's
          loadW2c(p * cpp, w2Bytes);
          if(p + 1 < a.parts) loadW1(p + 1);
          for(int c = 1; c < cpp; c++) loadW2c(p * cpp + c, w2Bytes);
          // the first part of the next tile comes after this tile's last chunk of GEMM2: the second epilogue can then
          // start as soon as the first one ends, and GEMM1 of the next tile runs underneath it
          if(p + 1 == a.parts && t + grid < numTiles) { loadA1(t + grid); loadW1(0); }
        }
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, PP_ERR_PRODUCER); }
    }
  }
  else if(warp == 1) {
    // ---------------- MMA issuer ----------------
    if(lane == 0) {
      const uint32_t descHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
      const uint32_t a1Lo = ((smemU32(sA1) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t a2Lo = ((smemU32(sA2) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t b1Lo = ((smemU32(sB1) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t b2Lo = ((smemU32(sB2) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t chunk16 = (uint32_t)PP_CHUNK >> 4, b1Slot16 = (uint32_t)a.b1Slot >> 4, b2Slot16 = (uint32_t)a.b2Slot >> 4;
      uint32_t s1 = 0, ph1 = 0, s2 = 0, ph2 = 0;
      bool ok = true;
      uint32_t G1n = 0;   // GEMM1 parts issued so far (over all tiles): phase of the d1 barriers
      uint32_t GC = 0;    // GEMM2 chunks issued so far: operand buffer GC & 1 and its barrier phases
      uint32_t tilesA = 0;  // tiles whose A operand has been waited for
      uint32_t itD2 = 0;    // tiles whose second accumulator has been started
      auto g1 = [&](bool firstOfTile, bool lastOfTile) {
        if(!ok) return;
        if(firstOfTile) {
          if(!mbarWait(smemU32(a1Full), tilesA & 1u, abortFlag)) { ok = false; return; }
          tilesA++;
        }
        PPT(true, G1n * 4);
        if(!mbarWait(smemU32(d1Empty), (G1n & 1u) ^ 1u, abortFlag)) { ok = false; return; }
        PPT(true, G1n * 4 + 1);
        tcFenceAfter();
        uint32_t acc = 0;
        for(int kc = 0; kc < a.kc1; kc++) {
          if(!mbarWait(smemU32(&b1Full[s1]), ph1, abortFlag)) { ok = false; return; }
          tcFenceAfter();
          const uint32_t aT = a1Lo + (uint32_t)kc * chunk16, bT = b1Lo + s1 * b1Slot16;
#pragma unroll
          for(int k = 0; k < 4; k++) { ummaLoHi(tmemBase + d1Col, aT + 2 * k, bT + 2 * k, descHi, a.idesc1, acc); acc = 1; }
          ummaCommit(smemU32(&b1Empty[s1]));
          if(++s1 == (uint32_t)a.numB1) { s1 = 0; ph1 ^= 1u; }
        }
        ummaCommit(smemU32(d1Full));
        if(lastOfTile) ummaCommit(smemU32(a1Empty));
        PPT(true, G1n * 4 + 2);
        G1n++;
      };
      auto g2 = [&](bool firstOfTile, bool lastOfTile) {
        if(!ok) return;
        const uint32_t buf = GC & 1u;
        PPT(true, 256 + GC * 4);
        if(!mbarWait(smemU32(&a2Full[buf]), (GC >> 1) & 1u, abortFlag)) { ok = false; return; }
        PPT(true, 256 + GC * 4 + 1);
        if(firstOfTile) {
          if(!mbarWait(smemU32(d2Empty), (itD2 & 1u) ^ 1u, abortFlag)) { ok = false; return; }
          itD2++;
        }
        const bool shared = a.numB2 == 0;
        if(!mbarWait(smemU32(shared ? &b1Full[s1] : &b2Full[s2]), shared ? ph1 : ph2, abortFlag)) { ok = false; return; }
        PPT(true, 256 + GC * 4 + 2);
        tcFenceAfter();
        const uint32_t aT = a2Lo + buf * chunk16, bT = shared ? b1Lo + s1 * b1Slot16 : b2Lo + s2 * b2Slot16;
#pragma unroll
        for(int k = 0; k < 4; k++) ummaLoHi(tmemBase + d2Col, aT + 2 * k, bT + 2 * k, descHi, a.idesc2, (firstOfTile && k == 0) ? 0u : 1u);
        if(shared) {
          ummaCommit(smemU32(&b1Empty[s1]));
          if(++s1 == (uint32_t)a.numB1) { s1 = 0; ph1 ^= 1u; }
        }
        else {
          ummaCommit(smemU32(&b2Empty[s2]));
          if(++s2 == (uint32_t)a.numB2) { s2 = 0; ph2 ^= 1u; }
        }
        ummaCommit(smemU32(&a2Empty[buf]));
        if(lastOfTile) ummaCommit(smemU32(d2Full));
        GC++;
      };
      int t = (int)blockIdx.x;
      if(t < numTiles) g1(true, a.parts == 1);
      for(; t < numTiles && ok; t += grid) {
        for(int p = 0; p < a.parts && ok; p++) {
          g2(p == 0, false);
          if(p + 1 < a.parts) g1(false, p + 2 == a.parts);
          for(int c = 1; c < cpp; c++) g2(false, p + 1 == a.parts && c + 1 == cpp);
          if(p + 1 == a.parts && t + grid < numTiles) g1(true, a.parts == 1);
        }
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, PP_ERR_MMA); }
    }
  }
  else {
    // ---------------- Epilogue: TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int cg = (warp - 2) >> 2;
    const int ew = warp - 2;
    uint8_t* sR = sStage + (size_t)ew * 3 * PP_UNIT;  // two residual / raw units, then one unit for the activated output
    uint8_t* sO = sR + 2 * PP_UNIT;
    uint64_t* myRes = resFull + ew * 2;
    const int U2 = a.Cn / 32;          // units of the second epilogue
    const int sw64 = (lane >> 1) & 3;  // 64-byte swizzle of the staging units
    const int sw128 = lane & 7;        // 128-byte swizzle of the operand buffer (row index modulo 8 = lane modulo 8)
    bool alive = true;
    uint32_t rs = 0;   // residual units consumed so far: ring slot rs % 2, phase (rs / 2) & 1
    uint32_t P = 0, it = 0;
    // the sequence of this warp's residual units: (tile, part, unit in part) with unit % PP_CG == cg
    int nt = (int)blockIdx.x, np = 0, nj = cg - PP_CG;   // the unit before the first one
    auto fetchNext = [&](uint32_t slotSeq) {
      // lane 0: request the residual of the next unit of this warp's sequence into ring slot slotSeq % 2
      nj += PP_CG;
      if(nj >= UP) { nj = cg; if(++np >= a.parts) { np = 0; nt += grid; } }
      if(nt >= numTiles) return;
      const uint32_t b = slotSeq & 1u;
      mbarExpectTx(smemU32(&myRes[b]), (uint32_t)PP_UNIT);
      tmaLoad2d(smemU32(sR + (size_t)b * PP_UNIT), &tmS, np * a.NP + nj * 32, nt * PP_BM + q * 32, smemU32(&myRes[b]));
    };
    gridDepWait();
    if(lane == 0) fetchNext(0);
    __syncwarp();
    for(int t = (int)blockIdx.x; t < numTiles && alive; t += grid, it++) {
      const int m0 = t * PP_BM;
      const int m = m0 + q * 32 + lane;
      const float mk = a.mask[m];
      const bool on = mk == 1.0f;
      // ---- first epilogue: parts of GEMM1 ----
      for(int p = 0; p < a.parts && alive; p++, P++) {
        PPT(threadIdx.x == 64, 512 + P * 16);
        bool ok = mbarWait(smemU32(d1Full), P & 1u, abortFlag);
        ok = __all_sync(0xffffffffu, ok);
        if(!ok) { alive = false; break; }
        PPT(threadIdx.x == 64, 512 + P * 16 + 1);
        tcFenceAfter();
        for(int j = cg; j < UP && alive; j += PP_CG) {
          const uint32_t slot = rs & 1u;
          const int uix = (j - cg) / PP_CG;
          PPT(threadIdx.x == 64, 512 + P * 16 + 2 + uix * 6);
          uint32_t r[32];
          tmemLd32(tmemBase + d1Col + (uint32_t)(j * 32) + ((uint32_t)(q * 32) << 16), r);
          // the slot of the unit after this one held this warp's store before last: it must have been read; then the
          // next residual is requested, so that its latency hides behind this unit's arithmetic
          if(lane == 0) { bulkWaitRead0(); fetchNext(rs + 1u); }
          __syncwarp();
          bool landed = mbarWait(smemU32(&myRes[slot]), (rs >> 1) & 1u, abortFlag);
          if(!__all_sync(0xffffffffu, landed)) { alive = false; break; }
          tmemLdWait();
          PPT(threadIdx.x == 64, 512 + P * 16 + 2 + uix * 6 + 1);
          if(j + PP_CG >= UP) {
            // this warp's last load of the part: the accumulator may be overwritten by the next part
            tcFenceBefore();
            __syncwarp();
            if(lane == 0) mbarArrive(smemU32(d1Empty));
          }
          const int c = p * a.NP + j * 32;  // first output channel of this unit
          float2 v[16];
#pragma unroll
          for(int k = 0; k < 16; k++) v[k] = make_float2(__uint_as_float(r[2 * k]), __uint_as_float(r[2 * k + 1]));
          uint8_t* rRow = sR + (size_t)slot * PP_UNIT + lane * 64;
#pragma unroll
          for(int jj = 0; jj < 4; jj++) {
            const uint4 x = *reinterpret_cast<const uint4*>(rRow + ((jj ^ sw64) << 4));
            const uint32_t xu[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for(int k = 0; k < 4; k++) v[4 * jj + k] = Pack2<T>::addTo(xu[k], v[4 * jj + k]);
          }
          // updated stream: in place of the residual, then out by TMA
#pragma unroll
          for(int jj = 0; jj < 4; jj++) {
            uint4 o;
            o.x = Pack2<T>::pack(v[4 * jj].x, v[4 * jj].y); o.y = Pack2<T>::pack(v[4 * jj + 1].x, v[4 * jj + 1].y);
            o.z = Pack2<T>::pack(v[4 * jj + 2].x, v[4 * jj + 2].y); o.w = Pack2<T>::pack(v[4 * jj + 3].x, v[4 * jj + 3].y);
            *reinterpret_cast<uint4*>(rRow + ((jj ^ sw64) << 4)) = o;
          }
          // norm + activation + mask of the layer between the two convolutions
          uint32_t actP[16];
          {
            const float4* sp = reinterpret_cast<const float4*>(a.scale1 + c);
            const float4* bp = reinterpret_cast<const float4*>(a.bias1 + c);
#pragma unroll
            for(int hh = 0; hh < 2; hh++) {
              float2 x[8];
#pragma unroll
              for(int k = 0; k < 4; k++) {
                const float4 s4 = __ldg(sp + 4 * hh + k), b4 = __ldg(bp + 4 * hh + k);
                x[2 * k] = __ffma2_rn(v[8 * hh + 2 * k], make_float2(s4.x, s4.y), make_float2(b4.x, b4.y));
                x[2 * k + 1] = __ffma2_rn(v[8 * hh + 2 * k + 1], make_float2(s4.z, s4.w), make_float2(b4.z, b4.w));
              }
              actStaged2<ACT, 8>(x);
#pragma unroll
              for(int k = 0; k < 8; k++) actP[8 * hh + k] = on ? Pack2<T>::pack(x[k].x, x[k].y) : 0u;
            }
          }
          // K chunk of GEMM2 this unit belongs to: its buffer is free once the chunk two before it has been multiplied
          const uint32_t gc = P * (uint32_t)cpp + (uint32_t)(j >> 1), abuf = gc & 1u;
          PPT(threadIdx.x == 64, 512 + P * 16 + 2 + uix * 6 + 2);
          {
            bool e = mbarWait(smemU32(&a2Empty[abuf]), ((gc >> 1) & 1u) ^ 1u, abortFlag);
            if(!__all_sync(0xffffffffu, e)) { alive = false; break; }
          }
          PPT(threadIdx.x == 64, 512 + P * 16 + 2 + uix * 6 + 3);
          {
            uint8_t* aRow = sA2 + (size_t)abuf * PP_CHUNK + (size_t)(q * 32 + lane) * 128;
            const int col0 = (j & 1) * 4;
#pragma unroll
            for(int jj = 0; jj < 4; jj++)
              *reinterpret_cast<uint4*>(aRow + (((col0 + jj) ^ sw128) << 4)) = make_uint4(actP[4 * jj], actP[4 * jj + 1], actP[4 * jj + 2], actP[4 * jj + 3]);
          }
          fenceProxyAsync();
          __syncwarp();
          if(lane == 0) {
            mbarArrive(smemU32(&a2Full[abuf]));
            tmaStore2d(&tmS, smemU32(sR + (size_t)slot * PP_UNIT), c, m0 + q * 32);
            bulkCommit();
          }
          PPT(threadIdx.x == 64, 512 + P * 16 + 2 + uix * 6 + 4);
          rs++;
        }
      }
      if(!alive) break;
      // ---- second epilogue: the next block's mid stream and its activated form ----
      {
        PPT(threadIdx.x == 64, 512 + (P - 1) * 16 + 14);
        bool ok = mbarWait(smemU32(d2Full), it & 1u, abortFlag);
        ok = __all_sync(0xffffffffu, ok);
        if(!ok) { alive = false; break; }
        PPT(threadIdx.x == 64, 512 + (P - 1) * 16 + 15);
        tcFenceAfter();
        for(int j = cg; j < U2; j += PP_CG) {
          uint32_t r[32];
          tmemLd32(tmemBase + d2Col + (uint32_t)(j * 32) + ((uint32_t)(q * 32) << 16), r);
          tmemLdWait();
          const int c = j * 32;
          float2 v[16];
#pragma unroll
          for(int k = 0; k < 16; k++) v[k] = make_float2(__uint_as_float(r[2 * k]), __uint_as_float(r[2 * k + 1]));
          uint32_t rawP[16], actP[16];
#pragma unroll
          for(int k = 0; k < 16; k++) rawP[k] = Pack2<T>::pack(v[k].x, v[k].y);
          {
            const float4* sp = reinterpret_cast<const float4*>(a.scale2 + c);
            const float4* bp = reinterpret_cast<const float4*>(a.bias2 + c);
#pragma unroll
            for(int hh = 0; hh < 2; hh++) {
              float2 x[8];
#pragma unroll
              for(int k = 0; k < 4; k++) {
                const float4 s4 = __ldg(sp + 4 * hh + k), b4 = __ldg(bp + 4 * hh + k);
                x[2 * k] = __ffma2_rn(v[8 * hh + 2 * k], make_float2(s4.x, s4.y), make_float2(b4.x, b4.y));
                x[2 * k + 1] = __ffma2_rn(v[8 * hh + 2 * k + 1], make_float2(s4.z, s4.w), make_float2(b4.z, b4.w));
              }
              actStaged2<ACT, 8>(x);
#pragma unroll
              for(int k = 0; k < 8; k++) actP[8 * hh + k] = on ? Pack2<T>::pack(x[k].x, x[k].y) : 0u;
            }
          }
          // staging: the ring slot that does not hold the residual requested ahead, and the third unit
          if(lane == 0) bulkWaitRead0();
          __syncwarp();
          uint8_t* rawRow = sR + (size_t)((rs + 1u) & 1u) * PP_UNIT + lane * 64;
          uint8_t* actRow = sO + lane * 64;
#pragma unroll
          for(int jj = 0; jj < 4; jj++) {
            *reinterpret_cast<uint4*>(rawRow + ((jj ^ sw64) << 4)) = make_uint4(rawP[4 * jj], rawP[4 * jj + 1], rawP[4 * jj + 2], rawP[4 * jj + 3]);
            *reinterpret_cast<uint4*>(actRow + ((jj ^ sw64) << 4)) = make_uint4(actP[4 * jj], actP[4 * jj + 1], actP[4 * jj + 2], actP[4 * jj + 3]);
          }
          fenceProxyAsync();
          __syncwarp();
          if(lane == 0) {
            tmaStore2d(&tmRaw2, smemU32(sR + (size_t)((rs + 1u) & 1u) * PP_UNIT), c, m0 + q * 32);
            tmaStore2d(&tmAct2, smemU32(sO), c, m0 + q * 32);
            bulkCommit();
          }
        }
        tcFenceBefore();
        __syncwarp();
        if(lane == 0) mbarArrive(smemU32(d2Empty));
      }
    }
    if(!alive && lane == 0 && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, PP_ERR_EPILOGUE); }
    if(lane == 0) bulkWaitAll();
  }

  // ---------------- common exit ----------------
  tcFenceBefore();
  __syncthreads();
  if(*abortFlag && threadIdx.x == 0 && !bad) {
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

typedef CUresult (*EncodeTiledFn2)(
  CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn2 encodeFn() {
  static EncodeTiledFn2 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn2>(p);
  });
  return fn;
}

static bool enc2d(CUtensorMap* tm, int dt, const void* base, uint64_t inner, uint64_t outer, uint64_t strideBytes, uint32_t boxInner, uint32_t boxOuter, CUtensorMapSwizzle sw) {
  EncodeTiledFn2 fn = encodeFn();
  if(!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {strideBytes};
  cuuint32_t box[2] = {boxInner, boxOuter};
  cuuint32_t estr[2] = {1, 1};
  return fn(tm, dt == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct ConvPostPrePlan {
  CUtensorMap tmA1, tmW1, tmW2, tmS, tmRaw2, tmAct2;
  PostPreArgs a;
  int dt, act, numSMs;
  size_t smemBytes;
};

typedef void (*PostPreKernelFn)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, PostPreArgs);
template <typename T>
static PostPreKernelFn postPreKernelForT(int act) {
  switch(act) {
    case KB_ACT_RELU: return convPostPreKernel<T, KB_ACT_RELU>;
    case KB_ACT_MISH: return convPostPreKernel<T, KB_ACT_MISH>;
    case KB_ACT_SILU: return convPostPreKernel<T, KB_ACT_SILU>;
    case KB_ACT_MISH_SCALE8: return convPostPreKernel<T, KB_ACT_MISH_SCALE8>;
    default: return convPostPreKernel<T, KB_ACT_IDENTITY>;
  }
}

// Part width of GEMM1: the largest multiple of 96 channels (whole 64-channel K chunks of GEMM2 per pair of 32-channel
// units, units divisible by the three epilogue warps of a quarter) that divides Ct and fits the tensor memory next to
// the accumulator of GEMM2.
static int postPrePartWidth(int Ct, int Cn) {
  for(int np = 192; np >= 192; np -= 96)
    if((Ct % np) == 0 && np + Cn <= 512) return np;
  return 0;
}

bool convPostPreEligible(int dt, int Cm, int Ct, int Cn) {
  if(dt != DT_F16 && dt != DT_BF16) return false;
  if((Cm % 64) != 0 || (Cn % 96) != 0 || Cn > 256 || Cn < 96) return false;
  const int NP = postPrePartWidth(Ct, Cn);
  if(NP == 0) return false;
  // shared memory: A1, two chunks of A2, three staging units per epilogue warp, two weight slots of GEMM1, one of GEMM2
  const long fixed = (long)(Cm / 64) * PP_CHUNK + 2L * PP_CHUNK + (long)PP_EPI_WARPS * 3 * PP_UNIT + PP_FIXED;
  return 227L * 1024 - fixed >= 3L * std::max(NP, Cn) * 128;
}

// in1: [rows][Cm] activated mid tensor; w1: [Ct][Cm]; stream: [rows][Ct] residual stream, updated in place; w2: [Cn][Ct];
// raw2 / act2: [rows][Cn].  All tensors dense (row stride = channel count) and 16-byte aligned.
ConvPostPrePlan* convPostPreCreate(
  int dt, const void* in1, int Cm, const void* w1, void* stream, int Ct, const float* scale1, const float* bias1, int act1,
  const void* w2, void* raw2, void* act2, int Cn, const float* scale2, const float* bias2, int act2code, const float* mask,
  int rowsPadMax) {
  if(!convPostPreEligible(dt, Cm, Ct, Cn) || act1 != act2code) return nullptr;
  ConvPostPrePlan* p = new ConvPostPrePlan();
  std::memset(&p->a, 0, sizeof(p->a));
  p->dt = dt; p->act = act1;
  PostPreArgs& a = p->a;
  a.NP = postPrePartWidth(Ct, Cn);
  a.Cm = Cm; a.Ct = Ct; a.Cn = Cn; a.parts = Ct / a.NP; a.kc1 = Cm / 64;
  a.b1Slot = std::max(a.NP, Cn) * 128; a.b2Slot = a.b1Slot;
  const long fixed = (long)a.kc1 * PP_CHUNK + 2L * PP_CHUNK + (long)PP_EPI_WARPS * 3 * PP_UNIT + PP_FIXED;
  // what shared memory is left goes to the rings: GEMM1 first (its parts are short bursts of kc1 slots), then GEMM2
  long left = 227L * 1024 - fixed;
  // One ring shared by both GEMMs (numB2 = 0) keeps the most loads in flight: measured on B200 for 192 -> 384 -> 192 with
  // three slots, shared 94 us per launch, split 2 + 1 105 us, 1 + 2 110 us.  KB_PP_RINGS="n1:n2" splits for experiments.
  a.numB1 = (int)std::min<long>(left / a.b1Slot, 8); a.numB2 = 0;
  if(const char* e = getenv("KB_PP_RINGS")) { int n1 = 0, n2 = 0; if(sscanf(e, "%d:%d", &n1, &n2) == 2 && n1 >= 1 && n2 >= 0 && (long)n1 * a.b1Slot + (long)n2 * a.b2Slot <= left) { a.numB1 = n1; a.numB2 = n2; } }
  p->smemBytes = (size_t)fixed + (size_t)a.numB1 * a.b1Slot + (size_t)a.numB2 * a.b2Slot;
  const uint32_t fmt = dt == DT_F16 ? 0u : 1u;
  a.idesc1 = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(a.NP >> 3) << 17) | ((uint32_t)(PP_BM >> 4) << 24);
  a.idesc2 = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(Cn >> 3) << 17) | ((uint32_t)(PP_BM >> 4) << 24);
  a.tmemCols = 512;
  a.scale1 = scale1; a.bias1 = bias1; a.scale2 = scale2; a.bias2 = bias2; a.mask = mask;
  const uint64_t rows = (uint64_t)rowsPadMax;
  bool ok = enc2d(&p->tmA1, dt, in1, (uint64_t)Cm, rows, (uint64_t)Cm * 2, 64, PP_BM, CU_TENSOR_MAP_SWIZZLE_128B) &&
            enc2d(&p->tmW1, dt, w1, (uint64_t)Cm, (uint64_t)Ct, (uint64_t)Cm * 2, 64, (uint32_t)a.NP, CU_TENSOR_MAP_SWIZZLE_128B) &&
            enc2d(&p->tmW2, dt, w2, (uint64_t)Ct, (uint64_t)Cn, (uint64_t)Ct * 2, 64, (uint32_t)Cn, CU_TENSOR_MAP_SWIZZLE_128B) &&
            enc2d(&p->tmS, dt, stream, (uint64_t)Ct, rows, (uint64_t)Ct * 2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B) &&
            enc2d(&p->tmRaw2, dt, raw2, (uint64_t)Cn, rows, (uint64_t)Cn * 2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B) &&
            enc2d(&p->tmAct2, dt, act2, (uint64_t)Cn, rows, (uint64_t)Cn * 2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
  if(!ok) { delete p; return nullptr; }
  int dev = 0, sms = 148;
  if(cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  p->numSMs = sms;
  return p;
}

void convPostPreDestroy(ConvPostPrePlan* p) { delete p; }

cudaError_t launchConvPostPre(cudaStream_t st, const ConvPostPrePlan* p, Geom g, int* statusWord) {
  PostPreArgs a = p->a;
  a.g = g;
  a.status = statusWord;
  const int numTiles = g.rowsPad / PP_BM;
  const int grid = numTiles < p->numSMs ? numTiles : p->numSMs;
  PostPreKernelFn fn = p->dt == DT_F16 ? postPreKernelForT<__half>(p->act) : postPreKernelForT<__nv_bfloat16>(p->act);
  {
    static std::mutex mu;
    static std::vector<std::pair<const void*, int>> done;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    const std::pair<const void*, int> key((const void*)fn, dev);
    if(std::find(done.begin(), done.end(), key) == done.end()) {
      cudaError_t e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if(e != cudaSuccess) return e;
      done.push_back(key);
    }
  }
  static const bool usePdl = getenv("KB_NO_PDL") == nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(PP_THREADS); cfg.dynamicSmemBytes = p->smemBytes; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  int numAttrs = 0;
  if(usePdl) {
    attr[numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[numAttrs].val.programmaticStreamSerializationAllowed = 1;
    numAttrs++;
  }
  cfg.attrs = attr; cfg.numAttrs = numAttrs;
  return cudaLaunchKernelEx(&cfg, fn, p->tmA1, p->tmW1, p->tmW2, p->tmS, p->tmRaw2, p->tmAct2, a);
}

}  // namespace kb

#ifdef KB_TC_TRACE
extern "C" int kb_debug_trace_pp(long long* out, int n) { return (int)cudaMemcpyFromSymbol(out, kb::g_ppTrace, sizeof(long long) * n); }
#endif
