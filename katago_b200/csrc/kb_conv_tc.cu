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
// Persistent CTAs (one per SM), 64 + 128*CG threads: warp 0 issues TMA loads, warp 1 owns TMEM and issues the
// MMAs, the remaining 4*CG warps run the epilogue (CG warps per TMEM lane quarter, taking 32-channel units in turn;
// CG = 2 by default, 3 for 1x1 convolutions whose epilogue is the critical path).
// Two accumulators live in TMEM, so the epilogue of tile i overlaps the main loop of tile i+1.
// Every wait is bounded: on time-out the kernel records a code in the status word and all roles
// leave through the common exit, which still frees TMEM.
#include "kb_conv_dev.cuh"
#include "kb_tile_table.h"

#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>
#include <algorithm>
#include <utility>

namespace kb {

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
  int pair;        // 1: CTA pairs (cluster of 2, cta_group::2 MMAs over 256 rows); bSlotBytes then holds half a weight tile
  // Per-tile dependencies (kernel variant DEPS): depCtr, if set, holds one counter per 128-row tile of the convolution
  // launched just before this one; a tile's inputs are ready when the counters of its row tile and both neighbours have
  // reached depTarget, and the kernel then does not wait for that whole grid.  doneCtr, if set, receives one increment
  // per epilogue warp and tile once that warp's stores of the tile have completed.
  const uint32_t* depCtr;
  uint32_t depTarget;
  uint32_t* doneCtr;
  int prefillB;    // request the first weight slots before waiting for the preceding kernels
  int residentB;   // 1x1 only: all weight tiles of this CTA's channel tile stay in shared memory for the whole kernel
  int jointAB;     // 1x1 with streamed weights: the activation chunk and the weight chunk of a K step share one "full"
                   // and one "empty" barrier (the rings have the same depth and advance together), so the MMA-issuing
                   // thread waits once and commits once per four MMAs; with a wait and a commit per operand that thread,
                   // not the tensor pipe, set the pace (about 1000 cycles per step where the MMAs need 480)
  uint32_t idesc;
  uint32_t tmemCols;
  int epiWarpBytes; // shared memory of one epilogue warp's staging units (TMA epilogue)
  int resRing;     // TMA epilogue with a residual: slots of each warp's residual ring (look-ahead = resRing - 1 units)
  int tmaEpi;      // 1: outputs and residual travel through shared memory and TMA (64-channel aligned ranges)
  int* status;     // device status word: 0 = ok
  int trace;       // timeline instrumentation requested (only in builds with KB_TC_TRACE)
  int tlSlot;      // whole-grid timeline slot + 1 (only in builds with KB_TC_TRACE)
};

// Optional timeline instrumentation (build with -DKB_TC_TRACE): CTA 0 of a launch whose shape matches the environment
// variable KB_TC_TRACE="k:inC:outC:hasResidual" records SM cycle counts of its producer, MMA and first epilogue warp.
// The same build also records a whole-grid timeline of up to TL_SLOTS consecutive launches (kb_debug_timeline_arm): per
// CTA the global-timer value (ns, common to all SMs) of a few events, the SM it ran on and its tile count.
#ifdef KB_TC_TRACE
__device__ long long g_tcTrace[2048];
#define TRACE(cond, slot) do { if((a.trace) && blockIdx.x == 0 && (cond)) g_tcTrace[(slot)] = clock64(); } while(0)
constexpr int TL_SLOTS = 12, TL_CTAS = 160, TL_EVENTS = 10;
__device__ unsigned long long g_tcTimeline[TL_SLOTS * TL_CTAS * TL_EVENTS];
// events: 0 CTA start, 1 first dependency satisfied (producer), 2 first MMA issued, 3 last MMA committed,
//         4 epilogue warp 2 finished its last tile, 5 CTA exit, 6 SM id, 7 tiles of this CTA,
//         8 / 9 SM cycle counter at events 2 / 3 (with the timer values: the SM clock while the MMAs ran)
#define TL(ev, val) do { if(a.tlSlot > 0 && blockIdx.x < TL_CTAS) g_tcTimeline[(((a.tlSlot - 1) * TL_CTAS) + blockIdx.x) * TL_EVENTS + (ev)] = (val); } while(0)
#define TLT(ev) TL(ev, globalTimerNs())
#else
#define TRACE(cond, slot) do { } while(0)
#define TL(ev, val) do { } while(0)
#define TLT(ev) do { } while(0)
#endif
constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
#ifndef KB_TC_EPI_CG
#define KB_TC_EPI_CG 2
#endif
// CG = epilogue warps per TMEM lane quarter (a template parameter of the kernel): the warps of a quarter take the
// 32-channel units of a tile in turn.  TC_EPI_CG is the default; convolutions whose epilogue is the critical path and
// whose units divide evenly run a variant with TC_EPI_CG_WIDE.
constexpr int TC_EPI_CG = KB_TC_EPI_CG;
constexpr int TC_EPI_CG_WIDE = 3;
constexpr int tcEpiWarps(int cg) { return 4 * cg; }
// deps: the kernel variant with per-tile dependencies carries one more warp, which polls the tile counters
constexpr int tcThreads(int cg, bool deps = false) { return 64 + 32 * 4 * cg + (deps ? 32 : 0); }

enum { TC_ERR_PRODUCER_TIMEOUT = 101, TC_ERR_MMA_TIMEOUT = 102, TC_ERR_EPILOGUE_TIMEOUT = 103 };

constexpr int tcMaxGroups(int cg) { return (16 + cg - 1) / cg; }  // 16-column groups per warp and tile (BN <= 256)

// One group of 16 output channels of one row: bias, residual (already in registers), raw store, norm+activation store.
template <typename T, int ACT>
__device__ __forceinline__ void epilogue16(
  const uint32_t (&r)[16], const Epilogue& ep, bool hasRes, const uint4& res0, const uint4& res1, int m, int c, float mk,
  const float* biasRow, const float* sScale, const float* sBias) {
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
  if(hasRes) {
    if(ep.resMask) {
#pragma unroll
      for(int j = 0; j < 16; j++) v[j] *= mk;
    }
    const uint32_t ru[8] = {res0.x, res0.y, res0.z, res0.w, res1.x, res1.y, res1.z, res1.w};
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

// All 16-column groups of one tile that belong to this warp (the warps of a quarter take the groups in turn).
// This is the path for channel ranges that the TMA epilogue cannot express (head convolutions, odd widths); it reads the
// residual and writes the outputs with plain vector accesses.
template <typename T, int ACT, int CG>
__device__ __forceinline__ void epilogueTile(
  const ConvTcArgs& a, uint32_t tmemAcc, int q, int cg, int m, int n0, float mk, const float* sScale, const float* sBias) {
  const Epilogue& ep = a.ep;
  const int b = min(m / a.g.PB, a.g.n - 1);
  const float* biasRow = ep.biasNC ? ep.biasNC + (size_t)b * a.outC : nullptr;
  const int groups = a.BN / 16;
  const bool hasRes = ep.residual != nullptr;
#pragma unroll
  for(int j = 0; j < tcMaxGroups(CG); j++) {
    const int gi = cg + CG * j;
    if(gi < groups) {
      uint32_t r[16];
      tmemLd16(tmemAcc + ((uint32_t)(q * 32) << 16) + (uint32_t)(gi * 16), r);
      uint4 res0 = make_uint4(0u, 0u, 0u, 0u), res1 = res0;
      if(hasRes) {
        const uint4* rp = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(ep.residual) + (size_t)m * ep.resStride + n0 + gi * 16);
        res0 = rp[0];
        res1 = rp[1];
      }
      tmemLdWait();
      epilogue16<T, ACT>(r, ep, hasRes, res0, res1, m, n0 + gi * 16, mk, biasRow, sScale, sBias);
    }
  }
}

#ifndef KB_TC_ACT_GROUP
#define KB_TC_ACT_GROUP 16
#endif
constexpr int TC_ACT_GROUP = KB_TC_ACT_GROUP;   // values per activation stage: independent chains covering the special-function latency
constexpr int TC_UNIT_BYTES = 32 * 64;        // one staging unit: 32 rows x 32 channels (64 B rows, 64-byte swizzle)
constexpr int tcMaxRing(int cg) { return (8 + cg - 1) / cg + 1; }  // BN <= 256 -> 8 units over the warps of a quarter, plus one

struct EpiWarp {
  uint8_t* sR;          // ring of `ring` units: the residual lands here, the raw output leaves from here
  uint8_t* sO;          // one unit for the activated output
  uint64_t* resFull;    // [ring] residual unit landed (TMA)
  int nU;               // units of this warp per tile
  int ring;             // slots of the residual/raw ring
  uint32_t seq;         // units processed so far, over all tiles
};

// Fetches the residual of this warp's unit number `seq` (counted over all of the CTA's tiles, nU per tile) into its
// ring slot, if that tile exists (lane 0 only).
// Which tiles a CTA works on: tile t covers rows (t / numNTiles) * rowsPerUnit + rowBase and channel tile t % numNTiles;
// a CTA takes t = first, first + step, ...  (a CTA pair shares t; rowBase selects the half).
struct TileMap {
  int first, step, numTiles, numNTiles, rowsPerUnit, rowBase;
  __device__ __forceinline__ int m0(int t) const { return (t / numNTiles) * rowsPerUnit + rowBase; }
  __device__ __forceinline__ int nTile(int t) const { return t % numNTiles; }
};

template <int CG>
__device__ __forceinline__ void prefetchResidual(
  const CUtensorMap* tmRes, const ConvTcArgs& a, const EpiWarp& es, uint32_t seq, const TileMap& tm, int q, int cg) {
  const int tile = tm.first + (int)(seq / (uint32_t)es.nU) * tm.step;
  if(tile >= tm.numTiles) return;
  const int j = (int)(seq % (uint32_t)es.nU);
  const int m0 = tm.m0(tile), n0 = tm.nTile(tile) * a.BN;
  const uint32_t b = seq % (uint32_t)es.ring;
  mbarExpectTx(smemU32(&es.resFull[b]), (uint32_t)TC_UNIT_BYTES);
  tmaLoad2d(smemU32(es.sR + (size_t)b * TC_UNIT_BYTES), tmRes, n0 + (cg + CG * j) * 32, m0 + q * 32, smemU32(&es.resFull[b]));
}

// Epilogue of one tile for one warp, staged through shared memory.  A warp owns 32 rows (its TMEM lane quarter) and
// every third 32-channel unit of the tile; each thread owns one row of a unit (64 contiguous bytes).  The residual
// unit was fetched by TMA one tile ahead; the updated residual stream overwrites it in place and goes back out by
// TMA; the activated tensor is staged in one more unit.  A unit is computed entirely in registers first; only then
// does the warp wait for the TMA engine to have read the previous unit's stores, so that wait is normally free.  All
// synchronisation is inside the warp, and global memory only sees whole 64-byte row segments written by the TMA engine.
// CHAIN: the tile belongs to a multi-layer launch (convChainKernel): residual units are fetched only within the tile
// (the caller requests the first ones once the tile's dependencies are known to be met), and a layer without a
// residual still advances the phase of the ring slot's barrier, so that slot and phase stay functions of es.seq when
// layers with and without a residual alternate.
template <typename T, int ACT, int CG, bool CHAIN = false>
__device__ __forceinline__ bool epilogueTileTma(
  const ConvTcArgs& a, const CUtensorMap* tmRaw, const CUtensorMap* tmAct, uint32_t tmemAcc, int q, int cg, int lane,
  int m0, int n0, float mk, const float* biasRow, EpiWarp& es, uint32_t tileIter, volatile int* abortFlag,
  const float* sScale, const float* sBias, const CUtensorMap* tmRes, const TileMap& tm, float rowScale, float& rowSumsq) {
  const Epilogue& ep = a.ep;
  const bool hasRes = ep.residual != nullptr;
  const int sw = (lane >> 1) & 3;  // 64-byte swizzle: 16-byte chunk index XOR bits 1..2 of the row
  const bool on = mk == 1.0f;
  // rotary embedding: this thread's board point; rows that are not board points turn by the angle of (0,0), which is 0
  float ropePx = 0.0f, ropePy = 0.0f;
  if(ACT == KB_ACT_ROPE_QK) {
    const int br = (m0 + q * 32 + lane) % a.g.PB;
    const int y = br / a.g.RW, x = br - y * a.g.RW;
    if(y < a.g.Y && x < a.g.X) { ropePx = (float)x; ropePy = (float)y; }
  }
  for(int j = 0; j < es.nU; j++) {
    const int u = cg + CG * j;
    const uint32_t slot = es.seq % (uint32_t)es.ring;
    TRACE(threadIdx.x == 64, 1024 + (int)(tileIter & 31u) * 16 + j * 5);
    uint32_t r[32];
    tmemLd32(tmemAcc + ((uint32_t)(q * 32) << 16) + (uint32_t)(u * 32), r);
    if(hasRes) {
      bool landed = mbarWait(smemU32(&es.resFull[slot]), (es.seq / (uint32_t)es.ring) & 1u, abortFlag);
      if(!__all_sync(0xffffffffu, landed)) return false;
    }
    tmemLdWait();
    TRACE(threadIdx.x == 64, 1024 + (int)(tileIter & 31u) * 16 + j * 5 + 1);
    const int c = n0 + u * 32;  // first output channel of this unit
    // the unit's 32 values of this row as 16 pairs: the arithmetic below uses the packed fp32 instructions
    float2 v[16];
#pragma unroll
    for(int k = 0; k < 16; k++) v[k] = make_float2(__uint_as_float(r[2 * k]), __uint_as_float(r[2 * k + 1]));
    if(ep.rowSumsq) {
      const float2 rs = make_float2(rowScale, rowScale);
#pragma unroll
      for(int k = 0; k < 16; k++) v[k] = __fmul2_rn(v[k], rs);
    }
    if(biasRow) {
      const float4* bp = reinterpret_cast<const float4*>(biasRow + c);
#pragma unroll
      for(int k = 0; k < 8; k++) {
        const float4 b4 = bp[k];
        v[2 * k] = __fadd2_rn(v[2 * k], make_float2(b4.x, b4.y));
        v[2 * k + 1] = __fadd2_rn(v[2 * k + 1], make_float2(b4.z, b4.w));
      }
    }
    uint8_t* rRow = es.sR + (size_t)slot * TC_UNIT_BYTES + lane * 64;
    if(hasRes) {
      if(ep.resMask) {
        const float2 mk2 = make_float2(mk, mk);
#pragma unroll
        for(int k = 0; k < 16; k++) v[k] = __fmul2_rn(v[k], mk2);
      }
#pragma unroll
      for(int jj = 0; jj < 4; jj++) {
        const uint4 x = *reinterpret_cast<const uint4*>(rRow + ((jj ^ sw) << 4));
        const uint32_t xu[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for(int k = 0; k < 4; k++) v[4 * jj + k] = Pack2<T>::addTo(xu[k], v[4 * jj + k]);
      }
    }
    if(ACT == KB_ACT_ROPE_QK && c < ep.ropeC1) {
      // v[k] is output channel pair c/2 + k; its two frequencies lie in shared memory (sScale holds ropeFreq), the
      // same address for every lane
      const float4* fq = reinterpret_cast<const float4*>(sScale + c);
#pragma unroll
      for(int k = 0; k < 8; k++) {
        const float4 f = fq[k];
        float sn0, cs0, sn1, cs1;
        __sincosf(fmaf(ropePy, f.y, ropePx * f.x), &sn0, &cs0);
        __sincosf(fmaf(ropePy, f.w, ropePx * f.z), &sn1, &cs1);
        const float2 t0 = v[2 * k], t1 = v[2 * k + 1];
        v[2 * k] = make_float2(t0.x * cs0 - t0.y * sn0, t0.x * sn0 + t0.y * cs0);
        v[2 * k + 1] = make_float2(t1.x * cs1 - t1.y * sn1, t1.x * sn1 + t1.y * cs1);
      }
    }
    const bool doRaw = ep.outRaw && c >= ep.rawC0 && c < ep.rawC1;
    const bool doAct = ep.outAct && c >= ep.actC0 && c < ep.actC1;
    // The raw output can go to its staging unit at once: with a residual it replaces the residual just read, without
    // one the two raw units alternate and the store from this one was waited for one unit ago.
    if(doRaw) {
      if(ep.sumsqOut) {
        // four running sums over the values k = 0, 1, 2, 3 (mod 4), as two pairs
        float2 s2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for(int k = 0; k < 16; k++) s2[k & 1] = __ffma2_rn(v[k], v[k], s2[k & 1]);
        rowSumsq += (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
      }
#pragma unroll
      for(int jj = 0; jj < 4; jj++) {
        uint4 o;
        o.x = Pack2<T>::pack(v[4 * jj].x, v[4 * jj].y); o.y = Pack2<T>::pack(v[4 * jj + 1].x, v[4 * jj + 1].y);
        o.z = Pack2<T>::pack(v[4 * jj + 2].x, v[4 * jj + 2].y); o.w = Pack2<T>::pack(v[4 * jj + 3].x, v[4 * jj + 3].y);
        *reinterpret_cast<uint4*>(rRow + ((jj ^ sw) << 4)) = o;
      }
    }
    uint32_t actP[16];
    if(ACT == KB_ACT_SWIGLU_PAIRS) {
      // columns 0..15 of the unit are "up" channels, 16..31 their "gate" channels: h = silu(up) * gate
      if(doAct) {
        const float2 kk2 = make_float2(-1.4426950408889634f, -1.4426950408889634f), one = make_float2(1.0f, 1.0f);
        float2 n[8];
#pragma unroll
        for(int k = 0; k < 8; k++) n[k] = __fmul2_rn(v[k], kk2);
#pragma unroll
        for(int k = 0; k < 8; k++) { n[k].x = ex2Approx(n[k].x); n[k].y = ex2Approx(n[k].y); }
#pragma unroll
        for(int k = 0; k < 8; k++) n[k] = __fadd2_rn(one, n[k]);
#pragma unroll
        for(int k = 0; k < 8; k++) { n[k].x = rcpApprox(n[k].x); n[k].y = rcpApprox(n[k].y); }
#pragma unroll
        for(int k = 0; k < 8; k++) n[k] = __fmul2_rn(__fmul2_rn(v[k], n[k]), v[8 + k]);
#pragma unroll
        for(int k = 0; k < 8; k++) actP[k] = Pack2<T>::pack(n[k].x, n[k].y);
      }
    }
    else if(doAct) {
      const int ca = c - ep.actC0;
      const float4* sp = reinterpret_cast<const float4*>(sScale + ca);
      const float4* bp = reinterpret_cast<const float4*>(sBias + ca);
      // all 32 values of the unit go through the activation stage by stage (TC_ACT_GROUP at a time)
      constexpr int G2 = TC_ACT_GROUP / 2;
#pragma unroll
      for(int hh = 0; hh < 32 / TC_ACT_GROUP; hh++) {
        float2 x[G2];
#pragma unroll
        for(int k = 0; k < G2 / 2; k++) {
          const float4 s4 = sp[(G2 / 2) * hh + k], b4 = bp[(G2 / 2) * hh + k];
          x[2 * k] = __ffma2_rn(v[G2 * hh + 2 * k], make_float2(s4.x, s4.y), make_float2(b4.x, b4.y));
          x[2 * k + 1] = __ffma2_rn(v[G2 * hh + 2 * k + 1], make_float2(s4.z, s4.w), make_float2(b4.z, b4.w));
        }
        actStaged2<ACT, G2>(x);
#pragma unroll
        for(int k = 0; k < G2; k++) actP[G2 * hh + k] = on ? Pack2<T>::pack(x[k].x, x[k].y) : 0u;
      }
    }
    TRACE(threadIdx.x == 64, 1024 + (int)(tileIter & 31u) * 16 + j * 5 + 2);
    // The TMA engine must have read the previous unit's stores before their staging units are written again; that
    // also frees the ring slot before this one for the residual of the same unit of the next tile.
    if(lane == 0) {
      bulkWaitRead0();
      // the slot of the unit before this one is free now: it takes the unit ring-1 ahead of this one
      if(CHAIN) {
        const int jn = j + es.ring - 1;
        if(hasRes && j > 0 && jn < es.nU) {
          const uint32_t b = (es.seq + (uint32_t)es.ring - 1u) % (uint32_t)es.ring;
          mbarExpectTx(smemU32(&es.resFull[b]), (uint32_t)TC_UNIT_BYTES);
          tmaLoad2d(smemU32(es.sR + (size_t)b * TC_UNIT_BYTES), tmRes, n0 + (cg + CG * jn) * 32, m0 + q * 32, smemU32(&es.resFull[b]));
        }
        if(!hasRes) mbarArrive(smemU32(&es.resFull[slot]));
      }
      else if(hasRes && es.seq > 0) prefetchResidual<CG>(tmRes, a, es, es.seq + (uint32_t)es.ring - 1u, tm, q, cg);
    }
    __syncwarp();
    TRACE(threadIdx.x == 64, 1024 + (int)(tileIter & 31u) * 16 + j * 5 + 3);
    if(doAct && ACT == KB_ACT_SWIGLU_PAIRS) {
      // 32 rows x 16 channels, 32-byte rows, no swizzle
      uint8_t* oRow = es.sO + lane * 32;
      *reinterpret_cast<uint4*>(oRow) = make_uint4(actP[0], actP[1], actP[2], actP[3]);
      *reinterpret_cast<uint4*>(oRow + 16) = make_uint4(actP[4], actP[5], actP[6], actP[7]);
    }
    else if(doAct) {
      uint8_t* oRow = es.sO + lane * 64;
#pragma unroll
      for(int jj = 0; jj < 4; jj++)
        *reinterpret_cast<uint4*>(oRow + ((jj ^ sw) << 4)) = make_uint4(actP[4 * jj], actP[4 * jj + 1], actP[4 * jj + 2], actP[4 * jj + 3]);
    }
    // make the generic-proxy writes visible to the TMA engine, then let lane 0 send the unit out
    fenceProxyAsync();
    __syncwarp();
    if(lane == 0) {
      if(doRaw) tmaStore2d(tmRaw, smemU32(es.sR + (size_t)slot * TC_UNIT_BYTES), c - ep.rawC0, m0 + q * 32);
      if(doAct) tmaStore2d(tmAct, smemU32(es.sO), ACT == KB_ACT_SWIGLU_PAIRS ? (c - ep.actC0) / 2 : c - ep.actC0, m0 + q * 32);
      bulkCommit();
    }
    TRACE(threadIdx.x == 64, 1024 + (int)(tileIter & 31u) * 16 + j * 5 + 4);
    es.seq++;
  }
  return true;
}

// One instantiation per element type, activation and epilogue kind: the epilogue is long straight-line code, and a
// kernel that carried every variant ran measurably slower (instruction cache).
template <typename T, int ACT, bool TMA_EPI, bool PAIR, int CG, bool DEPS>
__global__ void __launch_bounds__(tcThreads(CG, DEPS), 1) convTcKernel(
  const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmRes,
  const __grid_constant__ CUtensorMap tmRaw, const __grid_constant__ CUtensorMap tmAct, const ConvTcArgs a) {
  constexpr int TC_EPI_WARPS = tcEpiWarps(CG);
  constexpr int TC_MAX_RING = tcMaxRing(CG);
  extern __shared__ uint8_t smemRaw[];
  // 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smemA + (size_t)a.numA * a.aSlotBytes;
  uint8_t* smemR = smemB + (size_t)a.numB * a.bSlotBytes;  // epilogue staging (TMA epilogue only)
  float* sScale = reinterpret_cast<float*>(smemR + (TMA_EPI ? (size_t)TC_EPI_WARPS * a.epiWarpBytes : 0));
  float* sBias = sScale + 512;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sBias + 512);
  // barrier layout: fullA[numA] emptyA[numA] fullB[numB] emptyB[numB] accFull[2] accEmpty[2]
  uint64_t* fullA = bars;
  uint64_t* emptyA = fullA + a.numA;
  uint64_t* fullB = emptyA + a.numA;
  uint64_t* emptyB = fullB + a.numB;
  uint64_t* accFull = emptyB + a.numB;
  uint64_t* accEmpty = accFull + 2;
  uint64_t* resFull = accEmpty + 2;   // [TC_EPI_WARPS][TC_MAX_RING]
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(resFull + TC_EPI_WARPS * TC_MAX_RING);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);
  volatile int* gateTiles = abortFlag + 1;  // per-tile dependencies: how many of this CTA's tiles are known to be ready

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int numNTiles = a.outC / a.BN;
  const int taps = a.kY * a.kX;
  // CTA pair: both CTAs walk the same tile list; a tile is 256 rows, the even CTA (leader) takes the upper 128
  const uint32_t rank = PAIR ? clusterCtaRank() : 0u;
  const bool leader = rank == 0u;
  TileMap tm;
  tm.first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  tm.step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  tm.numNTiles = numNTiles;
  tm.rowsPerUnit = PAIR ? 2 * TC_BM : TC_BM;
  tm.numTiles = (a.g.rowsPad / tm.rowsPerUnit) * numNTiles;
  tm.rowBase = (int)rank * TC_BM;
  const int numTiles = tm.numTiles;

  gridDepLaunch();
  if(threadIdx.x == 0) {
    TLT(0);
#ifdef KB_TC_TRACE
    { unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid)); TL(6, (unsigned long long)smid); }
    { int nt = 0; for(int t = tm.first; t < numTiles; t += tm.step) nt++; TL(7, (unsigned long long)nt); }
#endif
    for(int s = 0; s < a.numA; s++) { mbarInit(smemU32(&fullA[s]), 1); mbarInit(smemU32(&emptyA[s]), 1); }
    for(int s = 0; s < a.numB; s++) { mbarInit(smemU32(&fullB[s]), 1); mbarInit(smemU32(&emptyB[s]), 1); }
    // the leader's accumulator-drained barrier collects the epilogue warps of both CTAs of a pair
    for(int s = 0; s < 2; s++) { mbarInit(smemU32(&accFull[s]), 1); mbarInit(smemU32(&accEmpty[s]), PAIR ? 2 * TC_EPI_WARPS : TC_EPI_WARPS); }
    for(int s = 0; s < TC_EPI_WARPS * TC_MAX_RING; s++) mbarInit(smemU32(&resFull[s]), 1);
    *abortFlag = 0;
    *gateTiles = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 1) {
    if(PAIR) { tmemAllocPair(smemU32(tmemSlot), a.tmemCols); tmemRelinquishPair(); }
    else { tmemAlloc(smemU32(tmemSlot), a.tmemCols); tmemRelinquish(); }
  }
  // next layer's norm parameters: read once per CTA (weights: not produced by the preceding kernels)
  if(a.ep.outAct && a.ep.scale) {
    const int nAct = a.ep.actC1 - a.ep.actC0;
    for(int i = threadIdx.x; i < nAct; i += blockDim.x) { sScale[i] = a.ep.scale[i]; sBias[i] = a.ep.bias[i]; }
  }
  if(ACT == KB_ACT_ROPE_QK) {
    // rotary frequencies of the query and key channels (up to 1024 floats: the scale and bias arrays together)
    for(int i = threadIdx.x; i < a.ep.ropeC1; i += blockDim.x) sScale[i] = a.ep.ropeFreq[i];
  }
  tcFenceBefore();
  __syncthreads();
  if(PAIR) clusterSync();  // the other CTA's barriers are initialised before anything here signals them
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  if(warp == 0) {
    // ---------------- TMA producer ----------------
    if(lane == 0) {
      uint32_t sa = 0, phA = 0, sb = 0, phB = 0;
      bool ok = true;
      // In a pair both CTAs load their own rows of A and their own half of each weight tile; every load signals the
      // leader's barrier, on which the leader alone has announced the bytes of both CTAs.
      const uint32_t aBytes = (PAIR ? 2u : 1u) * (uint32_t)a.aSlotBytes, bBytes = (PAIR ? 2u : 1u) * (uint32_t)a.bSlotBytes;
      const int bRow0 = PAIR ? (int)rank * (a.BN / 2) : 0;
      auto loadA = [&](uint32_t slot, int kc, int m0) {
        const uint32_t bar = smemU32(&fullA[slot]), dst = smemU32(smemA + (size_t)slot * a.aSlotBytes);
        if(leader) mbarExpectTx(bar, aBytes);
        if(PAIR) tmaLoad2dPair(dst, &tmA, kc * TC_BK, m0 - a.haloPad, pairLeaderAddr(bar));
        else tmaLoad2d(dst, &tmA, kc * TC_BK, m0 - a.haloPad, bar);
      };
      auto loadB = [&](uint32_t slot, int kc, int row) {
        const uint32_t bar = smemU32(&fullB[slot]), dst = smemU32(smemB + (size_t)slot * a.bSlotBytes);
        if(leader) mbarExpectTx(bar, bBytes);
        if(PAIR) tmaLoad2dPair(dst, &tmB, kc * TC_BK, row + bRow0, pairLeaderAddr(bar));
        else tmaLoad2d(dst, &tmB, kc * TC_BK, row, bar);
      };
      if(a.residentB) {
        // the number of CTAs (pairs) is a multiple of the number of channel tiles, so this CTA always works on the same one
        const int n0 = (tm.first % numNTiles) * a.BN;
        for(int kc = 0; kc < a.kChunks; kc++) loadB((uint32_t)kc, kc, n0);
      }
      // Weight ring: the first tile's first slots are requested before the wait on the preceding kernels as well (the
      // ring starts empty, so the slots need no empty-wait); the main loop below skips those loads.
      int prefilled = 0;
      if(!a.residentB && a.prefillB && !a.jointAB && tm.first < numTiles) {
        const int n0 = tm.nTile(tm.first) * a.BN;
        const int total = a.kChunks * taps;
        prefilled = a.numB < total ? a.numB : total;
        for(int i = 0; i < prefilled; i++) loadB((uint32_t)i, i / taps, (i % taps) * a.outC + n0);
      }
      // everything above touched only weights; the activations belong to the kernels before this one
      const bool tileDeps = DEPS && a.depCtr != nullptr;
      if(!tileDeps) gridDepWait();
      int issuedB = 0;  // weight slots of this CTA in issue order
      for(int t = tm.first; t < numTiles && ok; t += tm.step) {
        const int m0 = tm.m0(t), n0 = tm.nTile(t) * a.BN;
        if(tileDeps) {
          // the dependency warp polls the counters ahead of time and publishes how many tiles are ready
          const int need = (t - tm.first) / tm.step + 1;
          uint32_t spins = 0;
          while(*gateTiles < need) {
            if((++spins & 63u) == 0u && *abortFlag) { ok = false; break; }
          }
          if(!ok) break;
          asm volatile("fence.acq_rel.cta;" ::: "memory");
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        if(t == tm.first) TLT(1);
        for(int kc = 0; kc < a.kChunks && ok; kc++) {
          if(!mbarWait(smemU32(&emptyA[sa]), phA ^ 1u, abortFlag)) { ok = false; break; }
          TRACE(true, ((t - tm.first) / tm.step) * 16 + kc);
          if(!PAIR && a.jointAB) {
            // both operands of the step on the activation slot's barrier; the weight slot has the same index
            const uint32_t bar = smemU32(&fullA[sa]);
            mbarExpectTx(bar, aBytes + bBytes);
            tmaLoad2d(smemU32(smemA + (size_t)sa * a.aSlotBytes), &tmA, kc * TC_BK, m0 - a.haloPad, bar);
            tmaLoad2d(smemU32(smemB + (size_t)sa * a.bSlotBytes), &tmB, kc * TC_BK, n0, bar);
            if(++sa == (uint32_t)a.numA) { sa = 0; phA ^= 1u; }
            continue;
          }
          loadA(sa, kc, m0);
          if(++sa == (uint32_t)a.numA) { sa = 0; phA ^= 1u; }
          if(a.residentB) continue;
          for(int tap = 0; tap < taps; tap++, issuedB++) {
            if(issuedB >= prefilled) {
              if(!mbarWait(smemU32(&emptyB[sb]), phB ^ 1u, abortFlag)) { ok = false; break; }
              loadB(sb, kc, tap * a.outC + n0);
            }
            if(++sb == (uint32_t)a.numB) { sb = 0; phB ^= 1u; }
          }
        }
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_PRODUCER_TIMEOUT); }
    }
  }
  else if(warp == 1) {
    // ---------------- MMA issuer ----------------
    // One thread issues every MMA; its instruction stream is the critical path of the main loop, so the
    // descriptors are kept as 32-bit low words that only need an add per MMA, ring positions wrap by compare,
    // and the tap offsets are computed once.
    // In a pair only the leader issues; its MMAs read both CTAs' shared memory and write both CTAs' TMEM, and every
    // completion is signalled to the same barrier of both CTAs.
    if(lane == 0 && leader) {
      auto mma = [&](uint32_t d, uint32_t aLo, uint32_t bLo, uint32_t descHi, uint32_t acc) {
        if(PAIR) ummaLoHiPair(d, aLo, bLo, descHi, a.idesc, acc);
        else ummaLoHi(d, aLo, bLo, descHi, a.idesc, acc);
      };
      auto commit = [&](uint64_t* bar) {
        const uint32_t b = smemU32(bar);
        if(PAIR) { ummaCommitPair(b); ummaCommitPair(clusterMapAddr(b, 1u)); }
        else ummaCommit(b);
      };
      const uint32_t descHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);  // stride offset | version | SWIZZLE_128B
      const uint32_t aLoBase = ((smemU32(smemA) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t bLoBase = ((smemU32(smemB) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t aSlot16 = (uint32_t)a.aSlotBytes >> 4, bSlot16 = (uint32_t)a.bSlotBytes >> 4;
      // row offset of each tap inside the halo tile, in 16-byte units (one row = 128 B = 8 units)
      uint32_t tapOff[9];
#pragma unroll
      for(int tap = 0; tap < 9; tap++) {
        const int dy = tap / 3 - 1, dx = tap % 3 - 1;
        tapOff[tap] = (taps == 9) ? (uint32_t)(a.haloPad + dy * a.g.RW + dx) * 8u : 0u;
      }
      uint32_t sa = 0, phA = 0, sb = 0, phB = 0, it = 0;
      bool ok = true;
      for(int t = tm.first; t < numTiles && ok; t += tm.step, it++) {
        const uint32_t buf = it & 1u;
        // wait until the epilogue has drained this accumulator (two tiles ago)
        if(!mbarWait(smemU32(&accEmpty[buf]), ((it >> 1) & 1u) ^ 1u, abortFlag)) { ok = false; break; }
        tcFenceAfter();
        TRACE(true, 256 + it * 16);
        const uint32_t dTmem = tmemBase + buf * (uint32_t)a.BN;
        uint32_t accumulate = 0;
        for(int kc = 0; kc < a.kChunks && ok; kc++) {
          if(!mbarWait(smemU32(&fullA[sa]), phA, abortFlag)) { ok = false; break; }
          if(it == 0 && kc == 0) { TLT(2); TL(8, (unsigned long long)clock64()); }
          TRACE(true, 256 + it * 16 + 1 + kc);
          const uint32_t aLo = aLoBase + sa * aSlot16;
          if(taps == 9) {
#pragma unroll
            for(int tap = 0; tap < 9; tap++) {
              if(!mbarWait(smemU32(&fullB[sb]), phB, abortFlag)) { ok = false; break; }
              tcFenceAfter();
              const uint32_t aT = aLo + tapOff[tap], bT = bLoBase + sb * bSlot16;
#pragma unroll
              for(int k = 0; k < TC_BK / 16; k++) {
                // advancing K by 16 elements = 32 bytes = 2 units inside the 128-byte swizzle atom
                mma(dTmem, aT + 2 * k, bT + 2 * k, descHi, accumulate);
                accumulate = 1;
              }
              commit(&emptyB[sb]);  // frees the weight slot once these MMAs have read it
              if(++sb == (uint32_t)a.numB) { sb = 0; phB ^= 1u; }
            }
          }
          else if(a.residentB) {
            // weights were loaded once; the barrier of chunk kc completed its only phase during the first tile
            if(!mbarWait(smemU32(&fullB[kc]), 0u, abortFlag)) { ok = false; break; }
            tcFenceAfter();
            const uint32_t bT = bLoBase + (uint32_t)kc * bSlot16;
#pragma unroll
            for(int k = 0; k < TC_BK / 16; k++) {
              mma(dTmem, aLo + 2 * k, bT + 2 * k, descHi, accumulate);
              accumulate = 1;
            }
          }
          else if(!PAIR && a.jointAB) {
            // the weight chunk arrived on the same barrier as the activation chunk and is released with it below
            tcFenceAfter();
            const uint32_t bT = bLoBase + sa * bSlot16;
#pragma unroll
            for(int k = 0; k < TC_BK / 16; k++) {
              mma(dTmem, aLo + 2 * k, bT + 2 * k, descHi, accumulate);
              accumulate = 1;
            }
          }
          else {
            if(!mbarWait(smemU32(&fullB[sb]), phB, abortFlag)) { ok = false; break; }
            tcFenceAfter();
            const uint32_t bT = bLoBase + sb * bSlot16;
#pragma unroll
            for(int k = 0; k < TC_BK / 16; k++) {
              mma(dTmem, aLo + 2 * k, bT + 2 * k, descHi, accumulate);
              accumulate = 1;
            }
            commit(&emptyB[sb]);
            if(++sb == (uint32_t)a.numB) { sb = 0; phB ^= 1u; }
          }
          commit(&emptyA[sa]);
          if(++sa == (uint32_t)a.numA) { sa = 0; phA ^= 1u; }
        }
        if(ok) commit(&accFull[buf]);
        TLT(3);
        TL(9, (unsigned long long)clock64());
        TRACE(true, 256 + it * 16 + 15);
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_MMA_TIMEOUT); }
    }
  }
  else if(warp < 2 + TC_EPI_WARPS) {
    // ---------------- Epilogue: warps 2..; TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int cg = (warp - 2) >> 2;  // which of the quarter's warps: takes units cg, cg + CG, ...
    EpiWarp es;
    es.sR = smemR + (size_t)(warp - 2) * a.epiWarpBytes;
    es.sO = es.sR + (size_t)(a.epiWarpBytes - TC_UNIT_BYTES);
    es.resFull = resFull + (warp - 2) * TC_MAX_RING;
    es.nU = (a.BN / 32 - cg + CG - 1) / CG;
    es.ring = a.ep.residual ? a.resRing : 2;
    es.seq = 0;
    uint32_t it = 0;
    // mask, per-board bias, residual and the output buffers belong to the kernels before this one; with per-tile
    // dependencies nothing of a tile is written before the producer has seen its row tiles done (the accumulator
    // only fills after that), and the residual comes from a kernel further back, which has completed
    if(!(DEPS && a.depCtr != nullptr)) gridDepWait();
    int prevRowTile = -1;  // tile whose completion this warp still has to report
    for(int t = tm.first; t < numTiles; t += tm.step, it++) {
      const uint32_t buf = it & 1u;
      const int m0 = tm.m0(t), n0 = tm.nTile(t) * a.BN;
      // Nothing below depends on the accumulator yet: fetch mask and residual while the MMAs still run.
      TRACE(threadIdx.x == 64, 512 + it * 16);
      const int m = m0 + q * 32 + lane;
      const float mk = a.ep.mask ? a.ep.mask[m] : 1.0f;
      const int bIdx = min(m / a.g.PB, a.g.n - 1);
      const float* biasRow = a.ep.biasNC ? a.ep.biasNC + (size_t)bIdx * a.outC : nullptr;
      if(TMA_EPI) {
        if(a.ep.residual && lane == 0 && it == 0 && es.nU > 0) {
          // fill the ring; afterwards every unit that drains fetches the unit ring-1 ahead of it
          for(int k = 0; k < es.ring; k++) prefetchResidual<CG>(&tmRes, a, es, (uint32_t)k, tm, q, cg);
        }
        __syncwarp();
      }
      TRACE(threadIdx.x == 64, 512 + it * 16 + 1);
      bool ok = mbarWait(smemU32(&accFull[buf]), (it >> 1) & 1u, abortFlag);
      ok = __all_sync(0xffffffffu, ok);
      TRACE(threadIdx.x == 64, 512 + it * 16 + 2);
      if(!ok) {
        if(lane == 0 && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_EPILOGUE_TIMEOUT); }
        break;
      }
      tcFenceAfter();
      const uint32_t acc = tmemBase + buf * (uint32_t)a.BN;
      if(TMA_EPI) {
        float rowScale = 1.0f;
        if(a.ep.rowSumsq) {
          float ss = 0.0f;
          for(int k = 0; k < a.ep.rowSumsqSlots; k++) ss += a.ep.rowSumsq[(size_t)k * a.ep.sumsqRowStride + m];
          rowScale = mk == 1.0f ? rsqrtf(fmaf(ss, a.ep.rowInvC, a.ep.rowEps)) : 0.0f;
        }
        float rowSumsq = 0.0f;
        const bool ok2 = epilogueTileTma<T, ACT, CG>(a, &tmRaw, &tmAct, acc, q, cg, lane, m0, n0, mk, biasRow, es, it, abortFlag, sScale, sBias, &tmRes, tm, rowScale, rowSumsq);
        // this thread's partial sum of squares of row m: its own slot, a plain store (warps without units store 0)
        if(a.ep.sumsqOut) a.ep.sumsqOut[(size_t)(tm.nTile(t) * CG + cg) * a.ep.sumsqRowStride + m] = rowSumsq;
        if(!ok2) {
          if(lane == 0 && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_EPILOGUE_TIMEOUT); }
          break;
        }
      }
      else epilogueTile<T, ACT, CG>(a, acc, q, cg, m, n0, mk, sScale, sBias);
      // all TMEM reads of this warp are complete (tcgen05.wait::ld inside): hand the accumulator back
      tcFenceBefore();
      __syncwarp();
      TRACE(threadIdx.x == 64, 512 + it * 16 + 3);
      if(lane == 0) {
        if(PAIR) mbarArriveCluster(pairLeaderAddr(smemU32(&accEmpty[buf])));
        else mbarArrive(smemU32(&accEmpty[buf]));
      }
      if(DEPS && TMA_EPI && a.doneCtr != nullptr && lane == 0) {
        if(a.kY == 3) {
          // a 3x3 convolution's epilogue warps idle until the next accumulator is full: wait here for this tile's
          // stores to reach memory and report the tile at once
          bulkWaitAll();
          redReleaseGpuAdd(a.doneCtr + m0 / TC_BM, 1u);
        }
        else {
          // epilogue-bound kernels report one tile late: this tile's es.nU store groups may still be in flight,
          // everything older has reached memory
          if(prevRowTile >= 0) {
            bulkWaitPending(es.nU);
            redReleaseGpuAdd(a.doneCtr + prevRowTile, 1u);
          }
          prevRowTile = m0 / TC_BM;
        }
      }
    }
    if(lane == 0) bulkWaitAll();  // outstanding tile stores must complete before the CTA's shared memory goes away
    if(threadIdx.x == 64) TLT(4);
    if(DEPS && TMA_EPI && a.doneCtr != nullptr && lane == 0 && prevRowTile >= 0) {
      redReleaseGpuAdd(a.doneCtr + prevRowTile, 1u);
    }
  }
  else if(DEPS && lane == 0 && a.depCtr != nullptr) {
    // ---------------- dependency gate (its own warp: a thread that spins on global memory shares no instruction stream
    // with the producer) ----------------
    // The rows a tile reads (halo included) and the rows it will overwrite were last touched by the previous
    // convolution's row tiles rt-1 .. rt+1: wait for their counters, tile after tile, ahead of the producer.
    const int lastRowTile = a.g.rowsPad / TC_BM - 1;
    int ready = 0;
    for(int t = tm.first; t < numTiles; t += tm.step) {
      const int rt = tm.m0(t) / TC_BM;
      if(!waitTilesDone(a.depCtr, rt > 0 ? rt - 1 : 0, rt < lastRowTile ? rt + 1 : lastRowTile, a.depTarget, abortFlag, a.status)) {
        if(!*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, TC_ERR_PRODUCER_TIMEOUT); }
        break;
      }
      asm volatile("fence.acq_rel.cta;" ::: "memory");
      *gateTiles = ++ready;
    }
  }

  // ---------------- common exit ----------------
  // a kernel that ran on per-tile dependencies still completes only after the grid before it
  if(DEPS && a.depCtr != nullptr && threadIdx.x == 0) gridDepWait();
  tcFenceBefore();
  __syncthreads();
  if(*abortFlag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before the shared memory is released
    const uint64_t t0 = globalTimerNs();
    while(globalTimerNs() - t0 < 2000000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  // a pair leaves together: the leader's MMAs and commits touch the other CTA's shared memory, and the other CTA's
  // epilogue signals the leader's barriers
  if(PAIR) clusterSync();
  if(warp == 1) {
    tcFenceAfter();
    if(PAIR) tmemDeallocPair(tmemBase, a.tmemCols);
    else tmemDealloc(tmemBase, a.tmemCols);
  }
  if(threadIdx.x == 0) TLT(5);
}

// ---------------------------------------------------------------------------------------------
// Multi-layer launch ("chain"): one persistent grid runs several consecutive convolutions.
//
// A stand-alone launch pays, per CTA and layer, for its start-up (barriers, TMEM, first loads), for the epilogue of its
// last tile with the tensor pipe idle, for the hand-over of the SM to the next launch, and for the round of tiles that
// does not fill the machine.  Here a CTA never leaves: all tiles of all layers of the chain form one list that the CTAs
// take in turn (tile i of the list belongs to CTA i mod grid), so the epilogue of a layer's last tile overlaps the
// MMAs of the next layer's first one exactly as it does between two tiles of one layer, and the load balances over
// the whole chain instead of over each layer.
//
// What replaces the launch boundary: per-tile counters in global memory.  The epilogue warps of a tile add to the
// counter of its row tile once their stores have reached memory (red.release.gpu after cp.async.bulk.wait_group); the
// dependency warp of the CTA that will work on row tile r of the next layer waits until the counters of row tiles
// r-1, r, r+1 of the layer before have reached their target (the rows a 3x3 tile reads, and all readers of the rows
// it overwrites in buffers the blocks reuse), then lets the producer request that tile's loads.  A tile only ever
// waits for tiles earlier in the list and every CTA works through its part of the list in order, so with all CTAs
// resident (grid <= number of SMs, one CTA per SM) the waits cannot form a cycle; all of them are bounded like every
// other wait here.  The counters are zeroed by the host before the launch.
//
// Restrictions (the engine only builds chains that meet them): staged (TMA) epilogue, single CTAs, the same tile width
// and activation in every layer, per-layer tensor maps and arguments in device memory.

constexpr int CHAIN_MAX_LAYERS = 16;
struct alignas(128) ChainLayer {
  CUtensorMap tmA, tmB, tmRes, tmRaw, tmAct;
  ConvTcArgs a;  // a.g is replaced by the launch's geometry; ring sizes and slot strides come from ChainCfg
};
struct ChainCfg {
  int numLayers;
  Geom g;
  int numA, numB;        // ring depths, the same for every layer
  int aSlotStride;       // bytes between activation slots (>= the largest layer's halo tile)
  int bSlotStride;       // bytes between weight slots
  int epiWarpBytes;
  uint32_t tmemCols;
  int* status;
  int tlSlot;
};

template <typename T, int ACT>
__global__ void __launch_bounds__(tcThreads(TC_EPI_CG, true), 1) convChainKernel(const ChainLayer* __restrict__ layers, const ChainCfg c) {
  constexpr int CG = TC_EPI_CG;
  constexpr int TC_EPI_WARPS = tcEpiWarps(CG);
  constexpr int TC_MAX_RING = tcMaxRing(CG);
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smemA + (size_t)c.numA * c.aSlotStride;
  uint8_t* smemR = smemB + (size_t)c.numB * c.bSlotStride;
  ConvTcArgs* sArgs = reinterpret_cast<ConvTcArgs*>(smemR + (size_t)TC_EPI_WARPS * c.epiWarpBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sArgs + CHAIN_MAX_LAYERS);
  uint64_t* fullA = bars;
  uint64_t* emptyA = fullA + c.numA;
  uint64_t* fullB = emptyA + c.numA;
  uint64_t* emptyB = fullB + c.numB;
  uint64_t* accFull = emptyB + c.numB;
  uint64_t* accEmpty = accFull + 2;
  uint64_t* resFull = accEmpty + 2;   // [TC_EPI_WARPS][TC_MAX_RING]
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(resFull + TC_EPI_WARPS * TC_MAX_RING);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);
  volatile int* gateItems = abortFlag + 1;  // how many of this CTA's tiles (over all layers) have their dependencies met

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = (int)gridDim.x;
  const int rowTiles = c.g.rowsPad / TC_BM;
#ifdef KB_TC_TRACE
  struct { int trace, tlSlot; } a = {0, c.tlSlot};  // what the timeline macros look at
#endif

  gridDepLaunch();
  // every layer's arguments into shared memory (the roles read them in their inner loops)
  for(int i = threadIdx.x; i < c.numLayers * (int)(sizeof(ConvTcArgs) / 4); i += blockDim.x)
    reinterpret_cast<uint32_t*>(sArgs)[i] = reinterpret_cast<const uint32_t*>(&layers[i / (int)(sizeof(ConvTcArgs) / 4)].a)[i % (int)(sizeof(ConvTcArgs) / 4)];
  if(threadIdx.x == 0) {
    TLT(0);
#ifdef KB_TC_TRACE
    { unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid)); TL(6, (unsigned long long)smid); }
#endif
    for(int s = 0; s < c.numA; s++) { mbarInit(smemU32(&fullA[s]), 1); mbarInit(smemU32(&emptyA[s]), 1); }
    for(int s = 0; s < c.numB; s++) { mbarInit(smemU32(&fullB[s]), 1); mbarInit(smemU32(&emptyB[s]), 1); }
    for(int s = 0; s < 2; s++) { mbarInit(smemU32(&accFull[s]), 1); mbarInit(smemU32(&accEmpty[s]), TC_EPI_WARPS); }
    for(int s = 0; s < TC_EPI_WARPS * TC_MAX_RING; s++) mbarInit(smemU32(&resFull[s]), 1);
    *abortFlag = 0;
    *gateItems = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 1) { tmemAlloc(smemU32(tmemSlot), c.tmemCols); tmemRelinquish(); }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  // The list of this CTA's tiles: for L in layers, t = first(L), first(L) + grid, ... with first(L) chosen so that the
  // tiles of all layers, numbered through, go to the CTAs in turn.
  auto numTilesOf = [&](int L) { return rowTiles * (sArgs[L].outC / sArgs[L].BN); };
  auto firstOf = [&](int base) { int f = ((int)blockIdx.x - base) % grid; return f < 0 ? f + grid : f; };

  if(warp == 0) {
    // ---------------- TMA producer ----------------
    if(lane == 0) {
      uint32_t sa = 0, phA = 0, sb = 0, phB = 0;
      bool ok = true;
      int item = 0, base = 0;
      gridDepWait();  // the chain's inputs belong to the kernels before this launch
      for(int L = 0; L < c.numLayers && ok; L++) {
        const ConvTcArgs& la = sArgs[L];
        const CUtensorMap* tmA = &layers[L].tmA;
        const CUtensorMap* tmB = &layers[L].tmB;
        const int numTiles = numTilesOf(L), numNTiles = la.outC / la.BN, taps = la.kY * la.kX;
        const uint32_t aBytes = (uint32_t)la.aSlotBytes, bBytes = (uint32_t)la.bSlotBytes;
        for(int t = firstOf(base); t < numTiles && ok; t += grid, item++) {
          const int m0 = (t / numNTiles) * TC_BM, n0 = (t % numNTiles) * la.BN;
          {
            uint32_t spins = 0;
            while(*gateItems <= item) {
              if((++spins & 63u) == 0u && *abortFlag) { ok = false; break; }
            }
            if(!ok) break;
            asm volatile("fence.acq_rel.cta;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
          if(item == 0) TLT(1);
          for(int kc = 0; kc < la.kChunks && ok; kc++) {
            if(!mbarWait(smemU32(&emptyA[sa]), phA ^ 1u, abortFlag)) { ok = false; break; }
            {
              const uint32_t bar = smemU32(&fullA[sa]);
              mbarExpectTx(bar, aBytes);
              tmaLoad2d(smemU32(smemA + (size_t)sa * c.aSlotStride), tmA, kc * TC_BK, m0 - la.haloPad, bar);
            }
            if(++sa == (uint32_t)c.numA) { sa = 0; phA ^= 1u; }
            for(int tap = 0; tap < taps; tap++) {
              if(!mbarWait(smemU32(&emptyB[sb]), phB ^ 1u, abortFlag)) { ok = false; break; }
              const uint32_t bar = smemU32(&fullB[sb]);
              mbarExpectTx(bar, bBytes);
              tmaLoad2d(smemU32(smemB + (size_t)sb * c.bSlotStride), tmB, kc * TC_BK, tap * la.outC + n0, bar);
              if(++sb == (uint32_t)c.numB) { sb = 0; phB ^= 1u; }
            }
          }
        }
        base += numTiles;
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(c.status, 0, TC_ERR_PRODUCER_TIMEOUT); }
    }
  }
  else if(warp == 1) {
    // ---------------- MMA issuer ----------------
    if(lane == 0) {
      const uint32_t descHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
      const uint32_t aLoBase = ((smemU32(smemA) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t bLoBase = ((smemU32(smemB) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t aSlot16 = (uint32_t)c.aSlotStride >> 4, bSlot16 = (uint32_t)c.bSlotStride >> 4;
      uint32_t sa = 0, phA = 0, sb = 0, phB = 0, it = 0;
      bool ok = true;
      int base = 0;
      for(int L = 0; L < c.numLayers && ok; L++) {
        const ConvTcArgs& la = sArgs[L];
        const int numTiles = numTilesOf(L), taps = la.kY * la.kX, kChunks = la.kChunks, BN = la.BN;
        const uint32_t idesc = la.idesc;
        uint32_t tapOff[9];
#pragma unroll
        for(int tap = 0; tap < 9; tap++) {
          const int dy = tap / 3 - 1, dx = tap % 3 - 1;
          tapOff[tap] = (taps == 9) ? (uint32_t)(la.haloPad + dy * c.g.RW + dx) * 8u : 0u;
        }
        for(int t = firstOf(base); t < numTiles && ok; t += grid, it++) {
          const uint32_t buf = it & 1u;
          if(!mbarWait(smemU32(&accEmpty[buf]), ((it >> 1) & 1u) ^ 1u, abortFlag)) { ok = false; break; }
          tcFenceAfter();
          const uint32_t dTmem = tmemBase + buf * (uint32_t)BN;
          uint32_t accumulate = 0;
          for(int kc = 0; kc < kChunks && ok; kc++) {
            if(!mbarWait(smemU32(&fullA[sa]), phA, abortFlag)) { ok = false; break; }
            if(it == 0 && kc == 0) { TLT(2); TL(8, (unsigned long long)clock64()); }
            const uint32_t aLo = aLoBase + sa * aSlot16;
            if(taps == 9) {
#pragma unroll
              for(int tap = 0; tap < 9; tap++) {
                if(!mbarWait(smemU32(&fullB[sb]), phB, abortFlag)) { ok = false; break; }
                tcFenceAfter();
                const uint32_t aT = aLo + tapOff[tap], bT = bLoBase + sb * bSlot16;
#pragma unroll
                for(int k = 0; k < TC_BK / 16; k++) {
                  ummaLoHi(dTmem, aT + 2 * k, bT + 2 * k, descHi, idesc, accumulate);
                  accumulate = 1;
                }
                ummaCommit(smemU32(&emptyB[sb]));
                if(++sb == (uint32_t)c.numB) { sb = 0; phB ^= 1u; }
              }
            }
            else {
              if(!mbarWait(smemU32(&fullB[sb]), phB, abortFlag)) { ok = false; break; }
              tcFenceAfter();
              const uint32_t bT = bLoBase + sb * bSlot16;
#pragma unroll
              for(int k = 0; k < TC_BK / 16; k++) {
                ummaLoHi(dTmem, aLo + 2 * k, bT + 2 * k, descHi, idesc, accumulate);
                accumulate = 1;
              }
              ummaCommit(smemU32(&emptyB[sb]));
              if(++sb == (uint32_t)c.numB) { sb = 0; phB ^= 1u; }
            }
            ummaCommit(smemU32(&emptyA[sa]));
            if(++sa == (uint32_t)c.numA) { sa = 0; phA ^= 1u; }
          }
          if(ok) ummaCommit(smemU32(&accFull[buf]));
          TLT(3);
          TL(9, (unsigned long long)clock64());
          TL(7, (unsigned long long)(it + 1));
        }
        base += numTiles;
      }
      if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(c.status, 0, TC_ERR_MMA_TIMEOUT); }
    }
  }
  else if(warp < 2 + TC_EPI_WARPS) {
    // ---------------- Epilogue ----------------
    const int q = warp & 3;
    const int cg = (warp - 2) >> 2;
    EpiWarp es;
    es.sR = smemR + (size_t)(warp - 2) * c.epiWarpBytes;
    es.sO = es.sR + (size_t)(c.epiWarpBytes - TC_UNIT_BYTES);
    es.resFull = resFull + (warp - 2) * TC_MAX_RING;
    es.ring = 2;
    es.seq = 0;
    uint32_t it = 0;
    int base = 0;
    bool alive = true;
    TileMap tm = {};  // not used by the chain epilogue (it fetches residual units within the tile only)
    gridDepWait();
    for(int L = 0; L < c.numLayers && alive; L++) {
      const ConvTcArgs& la = sArgs[L];
      const CUtensorMap* tmRes = &layers[L].tmRes;
      const CUtensorMap* tmRaw = &layers[L].tmRaw;
      const CUtensorMap* tmAct = &layers[L].tmAct;
      const int numTiles = numTilesOf(L), numNTiles = la.outC / la.BN;
      es.nU = (la.BN / 32 - cg + CG - 1) / CG;
      const bool hasRes = la.ep.residual != nullptr;
      int prevRowTile = -1;  // tile of this layer whose completion this warp still has to report
      for(int t = firstOf(base); t < numTiles; t += grid, it++) {
        const uint32_t buf = it & 1u;
        const int m0 = (t / numNTiles) * TC_BM, n0 = (t % numNTiles) * la.BN;
        const int m = m0 + q * 32 + lane;
        const float mk = la.ep.mask ? la.ep.mask[m] : 1.0f;
        const int bIdx = min(m / c.g.PB, c.g.n - 1);
        const float* biasRow = la.ep.biasNC ? la.ep.biasNC + (size_t)bIdx * la.outC : nullptr;
        if(hasRes && lane == 0 && es.nU > 0) {
          // The residual may come from a layer of this chain: fetch it only once this tile's dependencies are known to
          // be met (they cover every row the residual unit holds).  The staging slots must be free as well.
          uint32_t spins = 0;
          bool gateOk = true;
          while(*gateItems <= (int)it) {
            if((++spins & 63u) == 0u && *abortFlag) { gateOk = false; break; }
          }
          if(gateOk) {
            asm volatile("fence.acq_rel.cta;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");
            bulkWaitRead0();
            for(int k = 0; k < es.ring && k < es.nU; k++) {
              const uint32_t b = (es.seq + (uint32_t)k) % (uint32_t)es.ring;
              mbarExpectTx(smemU32(&es.resFull[b]), (uint32_t)TC_UNIT_BYTES);
              tmaLoad2d(smemU32(es.sR + (size_t)b * TC_UNIT_BYTES), tmRes, n0 + (cg + CG * k) * 32, m0 + q * 32, smemU32(&es.resFull[b]));
            }
          }
        }
        __syncwarp();
        bool ok = mbarWait(smemU32(&accFull[buf]), (it >> 1) & 1u, abortFlag);
        ok = __all_sync(0xffffffffu, ok);
        if(!ok) {
          if(lane == 0 && !*abortFlag) { *abortFlag = 1; atomicCAS(c.status, 0, TC_ERR_EPILOGUE_TIMEOUT); }
          alive = false;
          break;
        }
        tcFenceAfter();
        const uint32_t acc = tmemBase + buf * (uint32_t)la.BN;
        float rowSumsq = 0.0f;
        const bool ok2 = epilogueTileTma<T, ACT, CG, true>(la, tmRaw, tmAct, acc, q, cg, lane, m0, n0, mk, biasRow, es, it, abortFlag, la.ep.scale, la.ep.bias, tmRes, tm, 1.0f, rowSumsq);
        if(!ok2) {
          if(lane == 0 && !*abortFlag) { *abortFlag = 1; atomicCAS(c.status, 0, TC_ERR_EPILOGUE_TIMEOUT); }
          alive = false;
          break;
        }
        tcFenceBefore();
        __syncwarp();
        if(lane == 0) mbarArrive(smemU32(&accEmpty[buf]));
        if(la.doneCtr != nullptr && lane == 0) {
          if(la.kY == 3) {
            // epilogue warps of a 3x3 layer idle until the next accumulator is full: report the tile at once
            bulkWaitAll();
            redReleaseGpuAdd(la.doneCtr + m0 / TC_BM, 1u);
          }
          else {
            // epilogue-bound layers report one tile late: this tile's stores may still be in flight
            if(prevRowTile >= 0) {
              bulkWaitPending(es.nU);
              redReleaseGpuAdd(la.doneCtr + prevRowTile, 1u);
            }
            prevRowTile = m0 / TC_BM;
          }
        }
      }
      if(la.doneCtr != nullptr && lane == 0 && prevRowTile >= 0) {
        bulkWaitAll();
        redReleaseGpuAdd(la.doneCtr + prevRowTile, 1u);
      }
      base += numTiles;
    }
    if(lane == 0) bulkWaitAll();
    if(threadIdx.x == 64) TLT(4);
  }
  else if(lane == 0) {
    // ---------------- dependency gate ----------------
    gridDepWait();
    const int lastRowTile = rowTiles - 1;
    int ready = 0, base = 0;
    bool ok = true;
    for(int L = 0; L < c.numLayers && ok; L++) {
      const ConvTcArgs& la = sArgs[L];
      const int numTiles = numTilesOf(L), numNTiles = la.outC / la.BN;
      for(int t = firstOf(base); t < numTiles; t += grid) {
        if(la.depCtr != nullptr) {
          const int rt = t / numNTiles;
          if(!waitTilesDone(la.depCtr, rt > 0 ? rt - 1 : 0, rt < lastRowTile ? rt + 1 : lastRowTile, la.depTarget, abortFlag, c.status)) {
            if(!*abortFlag) { *abortFlag = 1; atomicCAS(c.status, 0, TC_ERR_PRODUCER_TIMEOUT); }
            ok = false;
            break;
          }
        }
        asm volatile("fence.acq_rel.cta;" ::: "memory");
        *gateItems = ++ready;
      }
      base += numTiles;
    }
    if(!ok) *gateItems = 1 << 30;  // release the threads that spin on the gate; they leave through the abort flag
  }

  // ---------------- common exit ----------------
  tcFenceBefore();
  __syncthreads();
  if(*abortFlag && threadIdx.x == 0) {
    const uint64_t t0 = globalTimerNs();
    while(globalTimerNs() - t0 < 2000000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  if(warp == 1) {
    tcFenceAfter();
    tmemDealloc(tmemBase, c.tmemCols);
  }
  if(threadIdx.x == 0) TLT(5);
}

// ---------------------------------------------------------------------------------------------
// Host side

#ifdef KB_TC_TRACE
static int g_tlLaunch = 0, g_tlFirst = 1 << 30;  // tensor-core convolution launches since arming; first recorded launch
#endif

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

// Kernel variants by (element type, activation, epilogue kind).
typedef void (*ConvTcKernelFn)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, ConvTcArgs);
template <typename T, bool TMA_EPI, bool PAIR, int CG, bool DEPS>
static ConvTcKernelFn kernelForAct(int act) {
  switch(act) {
    case KB_ACT_RELU: return convTcKernel<T, KB_ACT_RELU, TMA_EPI, PAIR, CG, DEPS>;
    case KB_ACT_MISH: return convTcKernel<T, KB_ACT_MISH, TMA_EPI, PAIR, CG, DEPS>;
    case KB_ACT_SILU: return convTcKernel<T, KB_ACT_SILU, TMA_EPI, PAIR, CG, DEPS>;
    case KB_ACT_MISH_SCALE8: return convTcKernel<T, KB_ACT_MISH_SCALE8, TMA_EPI, PAIR, CG, DEPS>;
    // the SwiGLU epilogue exists with the default warp count and whole-grid dependencies only
    case KB_ACT_SWIGLU_PAIRS:
      if(DEPS) return nullptr;
      if(CG == TC_EPI_CG_WIDE) return (TMA_EPI && !PAIR) ? convTcKernel<T, KB_ACT_SWIGLU_PAIRS, true, false, TC_EPI_CG_WIDE, false> : nullptr;
      return convTcKernel<T, KB_ACT_SWIGLU_PAIRS, TMA_EPI, PAIR, TC_EPI_CG, false>;
    // so does the rotary epilogue, for single CTAs with the staged epilogue
    case KB_ACT_ROPE_QK:
      if(DEPS || !TMA_EPI || PAIR) return nullptr;
      return CG == TC_EPI_CG_WIDE ? convTcKernel<T, KB_ACT_ROPE_QK, true, false, TC_EPI_CG_WIDE, false> : convTcKernel<T, KB_ACT_ROPE_QK, true, false, TC_EPI_CG, false>;
    default: return convTcKernel<T, KB_ACT_IDENTITY, TMA_EPI, PAIR, CG, DEPS>;
  }
}
// The wide-epilogue variant exists for single CTAs with the staged epilogue only.
// The per-tile-dependency variant exists for single CTAs with the staged epilogue only.
template <typename T>
static ConvTcKernelFn kernelForT(int act, bool tmaEpi, bool pair, int cg, bool deps) {
  if(deps) {
    if(!tmaEpi || pair) return nullptr;
    return cg == TC_EPI_CG_WIDE ? kernelForAct<T, true, false, TC_EPI_CG_WIDE, true>(act)
                                : (cg == TC_EPI_CG ? kernelForAct<T, true, false, TC_EPI_CG, true>(act) : nullptr);
  }
  if(cg != TC_EPI_CG) return (tmaEpi && !pair && cg == TC_EPI_CG_WIDE) ? kernelForAct<T, true, false, TC_EPI_CG_WIDE, false>(act) : nullptr;
  if(pair) return tmaEpi ? kernelForAct<T, true, true, TC_EPI_CG, false>(act) : kernelForAct<T, false, true, TC_EPI_CG, false>(act);
  return tmaEpi ? kernelForAct<T, true, false, TC_EPI_CG, false>(act) : kernelForAct<T, false, false, TC_EPI_CG, false>(act);
}
static ConvTcKernelFn kernelFor(int dt, int act, bool tmaEpi, bool pair, int cg, bool deps) {
  return dt == DT_F16 ? kernelForT<__half>(act, tmaEpi, pair, cg, deps) : kernelForT<__nv_bfloat16>(act, tmaEpi, pair, cg, deps);
}

struct ConvTcPlan {
  CUtensorMap tmA, tmB;
  int dt, inC, outC, kY, kX, X, Y;
  int BN, kChunks, haloPad, aRows, aSlotBytes, bSlotBytes, numA, numB, residentB;
  int pair;  // CTA pairs: 256-row tiles, half a weight tile per CTA
  int cg;    // epilogue warps per TMEM lane quarter of the kernel variant this convolution runs
  uint32_t idesc, tmemCols;
  size_t smemBytes;
  int numSMs;
  int rowsPadMax;
  int tmaEpi, epiWarpBytes, resRing;
  CUtensorMap tmRes, tmRaw, tmAct;
};

static int pickBN(int k, int inC, int outC) {
  // experiments: KB_TC_BN="k:inC:outC=BN,..." overrides the table
  if(const char* e = getenv("KB_TC_BN")) {
    const char* s = e;
    while(*s) {
      int kk = 0, ic = 0, oc = 0, bn = 0, used = 0;
      if(sscanf(s, "%d:%d:%d=%d%n", &kk, &ic, &oc, &bn, &used) == 4) {
        if(kk == k && ic == inC && oc == outC && bn >= 16 && bn <= 256 && bn % 16 == 0 && outC % bn == 0) return bn;
        s += used;
      }
      while(*s && *s != ',') s++;
      if(*s == ',') s++;
    }
  }
  const TileRow r = tilePlanFor(k, inC, outC);
  return (r.BN > 0 && outC % r.BN == 0) ? r.BN : 0;
}

bool convTcEligible(int dt, int inC, int outC, int kY, int kX) {
  if(dt != DT_F16 && dt != DT_BF16) return false;
  if(!((kY == 1 && kX == 1) || (kY == 3 && kX == 3))) return false;
  if(inC % TC_BK != 0 || outC % 16 != 0) return false;
  return pickBN(kY, inC, outC) >= 16;
}

bool convTcRowNormEligible(int dt, int inC, int outC) {
  if(!convTcEligible(dt, inC, outC, 1, 1) || (outC % 32) != 0) return false;
  return (pickBN(1, inC, outC) % 32) == 0;
}

int convTcPlanRowSumSlots(const ConvTcPlan* p) {
  return (p && p->tmaEpi && (p->BN % 32) == 0) ? (p->outC / p->BN) * p->cg : 0;
}

int convTcRowSumSlots(int k, int inC, int outC) {
  const int bn = pickBN(k, inC, outC);
  // the staged epilogue needs whole 32-channel units
  return (bn > 0 && (bn % 32) == 0 && (outC % 32) == 0) ? (outC / bn) * TC_EPI_CG : 0;
}

bool convTcRopeEligible(int dt, int inC, int outC, int ropeC1) {
  // whole 32-channel units, frequencies in the kernel's 1024 floats of parameter space, single CTAs (the variant does
  // not exist for CTA pairs)
  if(!convTcRowNormEligible(dt, inC, outC) || ropeC1 <= 0 || ropeC1 > 1024 || (ropeC1 % 32) != 0) return false;
  return tilePlanFor(1, inC, outC).pair == 0;
}

bool convTcSwigluEligible(int dt, int inC, int F) {
  if(!convTcEligible(dt, inC, 2 * F, 1, 1) || (F % 16) != 0) return false;
  return (pickBN(1, inC, 2 * F) % 32) == 0;  // whole 32-column units, each holding 16 up and 16 gate channels
}

static bool encode2d(
  CUtensorMap* tm, int dt, const void* base, uint64_t inner, uint64_t outer, uint64_t strideBytes, uint32_t boxInner, uint32_t boxOuter,
  CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = getEncodeTiled();
  if(!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {strideBytes};
  cuuint32_t box[2] = {boxInner, boxOuter};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(
    tm, dt == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

constexpr int TC_FIXED_SMEM = 2 * 512 * 4 + 96 * 8 + 64 + 1024;  // norm parameters, barriers, TMEM slot, alignment slack

// Splits the shared memory between the weight ring and (optionally) the epilogue staging blocks.
static bool sizeRings(ConvTcPlan* p, int epiBytes) {
  const int budget = 227 * 1024 - TC_FIXED_SMEM - epiBytes;
  p->residentB = 0;
  if(p->kY == 1 && p->kX == 1) {
    // 1x1: little math per byte, so the kernel is bound by how many bytes of activations are in flight.  If all
    // weight tiles of one channel tile fit next to at least three activation slots they stay resident and only
    // activations stream; otherwise activation and weight slots are paired.
    const int allB = p->kChunks * p->bSlotBytes;
    if(allB + 3 * p->aSlotBytes <= budget && p->kChunks <= 12) {
      p->residentB = 1;
      p->numB = p->kChunks;
      int numA = (budget - allB) / p->aSlotBytes;
      p->numA = numA > 8 ? 8 : numA;
    }
    else {
      int n = budget / (p->aSlotBytes + p->bSlotBytes);
      if(n > 8) n = 8;
      if(n < 2) return false;
      p->numA = n;
      p->numB = n;
      // experiments: KB_TC_RING_1X1="a:b" sets the two ring depths separately where they fit
      if(const char* e = getenv("KB_TC_RING_1X1")) {
        int ra = 0, rb = 0;
        if(sscanf(e, "%d:%d", &ra, &rb) == 2 && ra >= 2 && rb >= 2 && ra <= 8 && rb <= 8 && ra * p->aSlotBytes + rb * p->bSlotBytes <= budget) {
          p->numA = ra; p->numB = rb;
        }
      }
    }
  }
  else {
    p->numA = 2;
    int numB = (budget - p->numA * p->aSlotBytes) / p->bSlotBytes;
    if(const char* e = getenv("KB_TC_NUMB")) { int v = atoi(e); if(v >= 1 && v <= 16) numB = v < numB ? v : numB; }
    if(numB > 12) numB = 12;
    if(numB < 2) return false;
    p->numB = numB;
  }
  p->smemBytes = (size_t)p->numA * p->aSlotBytes + (size_t)p->numB * p->bSlotBytes + (size_t)epiBytes + TC_FIXED_SMEM;
  return true;
}

ConvTcPlan* convTcCreate(
  int dt, const void* in, int inStride, int inC, const void* w, int outC, int kY, int kX, int X, int Y, int rowsPadMax) {
  if(!convTcEligible(dt, inC, outC, kY, kX)) return nullptr;
  if((inStride % 8) != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return nullptr;
  ConvTcPlan* p = new ConvTcPlan();
  p->dt = dt; p->inC = inC; p->outC = outC; p->kY = kY; p->kX = kX; p->X = X; p->Y = Y;
  p->rowsPadMax = rowsPadMax; p->tmaEpi = 0; p->cg = TC_EPI_CG;
  p->BN = pickBN(kY, inC, outC);
  p->kChunks = inC / TC_BK;
  const int maxShift = (kY == 3) ? (X + 1) + 1 : 0;  // RW + 1 rows up or down
  p->haloPad = (maxShift + 7) / 8 * 8;
  p->aRows = (p->haloPad + TC_BM + maxShift + 7) / 8 * 8;
  if(p->aRows > 256) { delete p; return nullptr; }
  // CTA pairs halve the weight bytes each SM stages and reads per MMA.  Measured on B200: a gain only for the widest
  // tiles (3x3 256->256, batch 512: 3 % faster, the SM clock under the power cap 3.5 % higher); the 192-wide tiles and
  // all 1x1 convolutions run 5-10 % slower in pairs (a 256-row MMA takes 143 cycles against 127 for 128 rows, and the
  // two CTAs move in lockstep).  KB_TC_PAIR=0/1 forces the choice for experiments.  Pairs need an even row-tile count,
  // which the padded-rows layout guarantees.
  bool wantPair = tilePlanFor(kY, inC, outC).pair != 0;
  if(const char* e = getenv("KB_TC_PAIR")) wantPair = atoi(e) != 0;
  p->pair = (wantPair && (rowsPadMax % (2 * TC_BM)) == 0 && (p->BN % 16) == 0) ? 1 : 0;
  p->aSlotBytes = p->aRows * 128;
  p->bSlotBytes = (p->pair ? p->BN / 2 : p->BN) * 128;
  if(!sizeRings(p, 0)) { delete p; return nullptr; }
  p->tmemCols = 32;
  while((int)p->tmemCols < 2 * p->BN) p->tmemCols *= 2;
  const uint32_t fmt = dt == DT_F16 ? 0u : 1u;
  // instruction descriptor: D=f32, A/B format, both K-major, N>>3 at bit 17, M>>4 at bit 24
  p->idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p->BN >> 3) << 17) | ((uint32_t)((p->pair ? 2 * TC_BM : TC_BM) >> 4) << 24);
  bool ok = encode2d(&p->tmA, dt, in, (uint64_t)inC, (uint64_t)rowsPadMax, (uint64_t)inStride * 2, TC_BK, (uint32_t)p->aRows) &&
            encode2d(&p->tmB, dt, w, (uint64_t)inC, (uint64_t)kY * kX * outC, (uint64_t)inC * 2, TC_BK, (uint32_t)(p->pair ? p->BN / 2 : p->BN));
  if(!ok) { delete p; return nullptr; }
  int dev = 0, sms = 148;
  if(cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  p->numSMs = sms;
  return p;
}

void convTcDestroy(ConvTcPlan* p) { delete p; }

// Decides how this convolution's outputs leave the SM.  When every output range (and the tile width) is a
// multiple of 32 channels the residual is fetched and the outputs are written by TMA through swizzled
// shared-memory units; otherwise the epilogue threads access global memory directly.
bool convTcSetEpilogue(ConvTcPlan* p, const Epilogue& ep) {
  p->tmaEpi = 0; p->cg = TC_EPI_CG;
  const bool force = getenv("KB_TC_NO_TMA_EPI") != nullptr && atoi(getenv("KB_TC_NO_TMA_EPI")) != 0;
  auto aligned32 = [](int c0, int c1) { return (c0 % 32) == 0 && (c1 % 32) == 0 && c1 > c0; };
  bool ok = !force && (p->BN % 32) == 0 && p->BN <= 256;
  if(ep.outRaw) ok = ok && aligned32(ep.rawC0, ep.rawC1) && (ep.rawStride % 8) == 0 && (reinterpret_cast<uintptr_t>(ep.outRaw) & 15) == 0;
  if(ep.outAct) ok = ok && aligned32(ep.actC0, ep.actC1) && (ep.actStride % 8) == 0 && (reinterpret_cast<uintptr_t>(ep.outAct) & 15) == 0;
  if(ep.residual) ok = ok && (ep.resStride % 8) == 0 && ep.resStride >= p->outC && (reinterpret_cast<uintptr_t>(ep.residual) & 15) == 0;
  const bool needsStaged = ep.act == KB_ACT_SWIGLU_PAIRS || ep.act == KB_ACT_ROPE_QK || ep.sumsqOut || ep.rowSumsq;
  if(!ok || (!ep.outRaw && !ep.outAct)) return needsStaged ? false : sizeRings(p, 0);
  // per warp: the residual/raw ring (one tile of this warp's units plus one with a residual, else two units) and one
  // unit for the activated output
  // With a residual the ring holds it one whole tile ahead for 1x1 convolutions, whose epilogue is the critical path;
  // a 3x3 convolution hides its epilogue behind the MMAs and does better with the shared memory spent on weight slots,
  // so it looks only one unit ahead.  Without a residual two raw units alternate (none if there is no raw output).
  // Twelve epilogue warps instead of eight where the epilogue is the critical path and the tile's units divide by
  // three: measured on B200, 1x1 192->384 with residual runs 11 % faster, 3x3 convolutions (which hide the epilogue
  // and lose weight slots to the staging units) 5 % slower.  KB_TC_WIDE_EPI=0 turns the variant off, =2 uses it for
  // every 1x1 convolution that qualifies.
  static const int wideMode = getenv("KB_TC_WIDE_EPI") ? atoi(getenv("KB_TC_WIDE_EPI")) : 1;
  p->cg = TC_EPI_CG;
  {
    const TileRow row = tilePlanFor(p->kY, p->inC, p->outC);
    const int want = wideMode > 1 ? TC_EPI_CG_WIDE : (ep.residual ? row.epiWarpsRes : row.epiWarps);
    // the 12-warp variant exists for single CTAs and 1x1 kernels, for the plain staged epilogue and for the SwiGLU and
    // rotary ones.  A tile's units need not divide by three (8 units: 3 + 3 + 2): every warp walks its own unit
    // sequence, residual ring included.
    const bool specialWide = (ep.act == KB_ACT_SWIGLU_PAIRS || ep.act == KB_ACT_ROPE_QK) && !ep.residual && !ep.sumsqOut;
    // a producer of row sums writes one slot per (channel tile, epilogue warp of the quarter): the consumer learns the
    // count from the plan (convTcPlanRowSumSlots), so the producer may have twelve warps as well
    const bool sumsWide = ep.sumsqOut && !ep.rowSumsq && ep.act != KB_ACT_SWIGLU_PAIRS && ep.act != KB_ACT_ROPE_QK;
    const bool plainWide = !needsStaged || sumsWide;
    if(TC_EPI_CG == 2 && wideMode > 0 && want == TC_EPI_CG_WIDE && p->kY == 1 && !p->pair && (plainWide || specialWide))
      p->cg = TC_EPI_CG_WIDE;
  }
  const int unitsPerWarp = (p->BN / 32 + p->cg - 1) / p->cg;
  p->resRing = (p->kY == 1) ? unitsPerWarp + 1 : 2;
  // A 1x1 convolution with a long K loop (FFN down: 1024 channels = 16 steps) is bound by how many operand steps are in
  // flight, not by its epilogue: three residual slots instead of four leave room for a fourth operand stage (measured
  // 68.4 -> 61.6 us; two slots 63.2 us).  KB_TC_RES_RING overrides for experiments.
  if(p->kY == 1 && p->kChunks >= 8 && p->resRing > 3) p->resRing = 3;
  if(const char* e = getenv("KB_TC_RES_RING")) {
    const int v = atoi(e);
    if(p->kY == 1 && v >= 2 && v <= unitsPerWarp + 1) p->resRing = v;
  }
  const int rawUnits = ep.residual ? p->resRing : (ep.outRaw ? 2 : 0);
  p->epiWarpBytes = (rawUnits + (ep.outAct ? 1 : 0)) * TC_UNIT_BYTES;
  if(!sizeRings(p, tcEpiWarps(p->cg) * p->epiWarpBytes)) { p->cg = TC_EPI_CG; return needsStaged ? false : sizeRings(p, 0); }
  const uint64_t rows = (uint64_t)p->rowsPadMax;
  const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_64B;
  bool enc = true;
  if(ep.residual) enc = enc && encode2d(&p->tmRes, p->dt, ep.residual, (uint64_t)p->outC, rows, (uint64_t)ep.resStride * 2, 32, 32, sw);
  if(ep.outRaw) enc = enc && encode2d(&p->tmRaw, p->dt, ep.outRaw, (uint64_t)(ep.rawC1 - ep.rawC0), rows, (uint64_t)ep.rawStride * 2, 32, 32, sw);
  if(ep.outAct && ep.act == KB_ACT_SWIGLU_PAIRS)
    enc = enc && encode2d(&p->tmAct, p->dt, ep.outAct, (uint64_t)(ep.actC1 - ep.actC0) / 2, rows, (uint64_t)ep.actStride * 2, 16, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
  else if(ep.outAct) enc = enc && encode2d(&p->tmAct, p->dt, ep.outAct, (uint64_t)(ep.actC1 - ep.actC0), rows, (uint64_t)ep.actStride * 2, 32, 32, sw);
  if(!enc) { p->cg = TC_EPI_CG; return needsStaged ? false : sizeRings(p, 0); }
  p->tmaEpi = 1;
  return true;
}

bool convTcDepsCapable(const ConvTcPlan* p) { return p && p->tmaEpi && !p->pair; }
int convTcKernelSize(const ConvTcPlan* p) { return p->kY; }
bool convTcChainPreferred(const ConvTcPlan* p) { return tilePlanFor(p->kY, p->inC, p->outC).chain != 0; }
int convTcDoneCount(const ConvTcPlan* p) { return (p->outC / p->BN) * tcEpiWarps(p->cg); }
int convTcGridSize(const ConvTcPlan* p, const Geom& g) {
  const int unitRows = p->pair ? 2 * TC_BM : TC_BM;
  const int maxUnits = p->pair ? p->numSMs / 2 : p->numSMs;
  const int numTiles = (g.rowsPad / unitRows) * (p->outC / p->BN);
  int units = numTiles < maxUnits ? numTiles : maxUnits;
  if(p->residentB) {
    const int nt = p->outC / p->BN;
    units = units / nt * nt;
    if(units < nt) units = nt;
  }
  return p->pair ? 2 * units : units;
}

cudaError_t launchConvTc(cudaStream_t st, const ConvTcPlan* p, Geom g, const Epilogue& ep, int* statusWord, const ConvTcDeps* deps) {
  // vector accesses in the epilogue need 16-byte aligned rows and 16-channel aligned ranges
  if(ep.outRaw && ((ep.rawStride % 8) || (ep.rawC0 % 16) || (ep.rawC1 % 16))) return cudaErrorInvalidValue;
  if(ep.outAct && ((ep.actStride % 8) || (ep.actC0 % 16) || (ep.actC1 % 16) || ((ep.actC1 - ep.actC0) > 512 && ep.act != KB_ACT_SWIGLU_PAIRS))) return cudaErrorInvalidValue;
  if(ep.residual && (ep.resStride % 8)) return cudaErrorInvalidValue;
  ConvTcArgs a;
  a.g = g; a.ep = ep;
  a.inC = p->inC; a.outC = p->outC; a.kY = p->kY; a.kX = p->kX;
  a.BN = p->BN; a.kChunks = p->kChunks; a.haloPad = p->haloPad; a.aRows = p->aRows;
  a.aSlotBytes = p->aSlotBytes; a.bSlotBytes = p->bSlotBytes; a.numA = p->numA; a.numB = p->numB; a.residentB = p->residentB;
  static const bool jointOff = getenv("KB_TC_NO_JOINT_AB") != nullptr && atoi(getenv("KB_TC_NO_JOINT_AB")) != 0;
  a.jointAB = (!jointOff && p->kY == 1 && p->kX == 1 && !p->residentB && !p->pair && p->numA == p->numB) ? 1 : 0;
  static const bool prefillB = getenv("KB_NO_B_PREFILL") == nullptr;
  a.prefillB = prefillB ? 1 : 0;
  a.pair = p->pair;
  a.depCtr = nullptr; a.depTarget = 0; a.doneCtr = nullptr;
  a.idesc = p->idesc; a.tmemCols = p->tmemCols;
  a.status = statusWord;
  a.trace = 0;
  a.tlSlot = 0;
#ifdef KB_TC_TRACE
  {
    const int idx = g_tlLaunch++;
    if(idx >= g_tlFirst && idx < g_tlFirst + TL_SLOTS) a.tlSlot = idx - g_tlFirst + 1;
  }
  if(const char* e = getenv("KB_TC_TRACE")) {
    int k = 0, ic = 0, oc = 0, r = 0;
    if(sscanf(e, "%d:%d:%d:%d", &k, &ic, &oc, &r) == 4 && k == p->kY && ic == p->inC && oc == p->outC && r == (ep.residual ? 1 : 0)) a.trace = 1;
  }
#endif
  a.tmaEpi = p->tmaEpi;
  a.epiWarpBytes = p->epiWarpBytes;
  a.resRing = p->resRing;
  // work units: tiles of 128 rows for single CTAs, of 256 rows for CTA pairs
  if(p->pair && (g.rowsPad % (2 * TC_BM)) != 0) return cudaErrorInvalidValue;
  const int unitRows = p->pair ? 2 * TC_BM : TC_BM;
  const int maxUnits = p->pair ? p->numSMs / 2 : p->numSMs;
  const int numTiles = (g.rowsPad / unitRows) * (p->outC / p->BN);
  int units = numTiles < maxUnits ? numTiles : maxUnits;
  if(p->residentB) {
    const int nt = p->outC / p->BN;
    units = units / nt * nt;  // each CTA (pair) keeps one channel tile
    if(units < nt) units = nt;
  }
  const int grid = p->pair ? 2 * units : units;
  // Programmatic dependent launch: the preamble (barriers, TMEM, resident weights) overlaps the tail of the kernel
  // before this one in the stream; the kernel waits for that kernel before it touches any activation.
  static const bool usePdl = getenv("KB_NO_PDL") == nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(tcThreads(p->cg)); cfg.dynamicSmemBytes = p->smemBytes; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int numAttrs = 0;
  if(p->pair) {
    attr[numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[numAttrs].val.clusterDim.x = 2; attr[numAttrs].val.clusterDim.y = 1; attr[numAttrs].val.clusterDim.z = 1;
    numAttrs++;
  }
  if(usePdl) {
    attr[numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[numAttrs].val.programmaticStreamSerializationAllowed = 1;
    numAttrs++;
  }
  cfg.attrs = attr; cfg.numAttrs = numAttrs;
  // without an activated output the activation code is irrelevant: use the identity variant
  // Per-tile dependencies: this launch reports its tiles if asked to, and waits per tile on the convolution before it
  // if that one reports and fills every SM (its CTAs can then only all have started once the kernels before it have
  // left the SMs, so at most these two grids overlap).
  bool useDeps = false;
  if(deps && convTcDepsCapable(p) && ep.act != KB_ACT_SWIGLU_PAIRS && ep.act != KB_ACT_ROPE_QK) {
    if(deps->done) { a.doneCtr = deps->done; useDeps = true; }
    if(deps->wait && deps->waitPlan && convTcDepsCapable(deps->waitPlan) && convTcGridSize(deps->waitPlan, g) == p->numSMs) {
      a.depCtr = deps->wait;
      a.depTarget = (uint32_t)convTcDoneCount(deps->waitPlan);
      useDeps = true;
    }
  }
  {
    static const int dbg = getenv("KB_TILE_DEPS_DEBUG") ? atoi(getenv("KB_TILE_DEPS_DEBUG")) : 0;
    if(dbg == 1) a.depCtr = nullptr;                       // report only
    if(dbg == 2) { a.doneCtr = nullptr; a.depTarget = 0; }  // poll only (always satisfied)
  }
  const int actVariant = ep.act == KB_ACT_ROPE_QK ? KB_ACT_ROPE_QK : (ep.outAct ? ep.act : KB_ACT_IDENTITY);
  ConvTcKernelFn fn = kernelFor(p->dt, actVariant, p->tmaEpi != 0, p->pair != 0, p->cg, useDeps);
  cfg.blockDim = dim3(tcThreads(p->cg, useDeps));
  if(!fn) return cudaErrorInvalidValue;
  {
    // opt in to the large dynamic shared memory once per variant and device
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
  return cudaLaunchKernelEx(&cfg, fn, p->tmA, p->tmB, p->tmRes, p->tmRaw, p->tmAct, a);
}

// ---------------------------------------------------------------------------------------------
// Multi-layer launches: host side

typedef void (*ConvChainKernelFn)(const ChainLayer*, ChainCfg);
template <typename T>
static ConvChainKernelFn chainKernelForT(int act) {
  switch(act) {
    case KB_ACT_RELU: return convChainKernel<T, KB_ACT_RELU>;
    case KB_ACT_MISH: return convChainKernel<T, KB_ACT_MISH>;
    case KB_ACT_SILU: return convChainKernel<T, KB_ACT_SILU>;
    case KB_ACT_MISH_SCALE8: return convChainKernel<T, KB_ACT_MISH_SCALE8>;
    default: return convChainKernel<T, KB_ACT_IDENTITY>;
  }
}

struct ConvChainPlan {
  ChainLayer* dLayers = nullptr;
  ChainCfg cfg;
  size_t smemBytes = 0;
  int dt = 0, act = 0, numSMs = 148, maxNTiles = 1;
};

int convTcTileWidth(const ConvTcPlan* p) { return p->BN; }

bool convChainEligible(const ConvTcPlan* p, const Epilogue& ep) {
  if(!p || !p->tmaEpi || p->pair) return false;
  if(ep.biasNC || ep.rowSumsq || ep.sumsqOut || ep.act == KB_ACT_SWIGLU_PAIRS || ep.act == KB_ACT_ROPE_QK) return false;
  if((p->BN % 32) != 0) return false;
  return true;
}

ConvChainPlan* convChainCreate(const ConvChainMember* members, int n) {
  if(n < 2 || n > CHAIN_MAX_LAYERS) return nullptr;
  ConvChainPlan* c = new ConvChainPlan();
  const ConvTcPlan* p0 = members[0].plan;
  c->dt = p0->dt;
  c->act = members[0].ep.outAct ? members[0].ep.act : KB_ACT_IDENTITY;
  c->numSMs = p0->numSMs;
  std::vector<ChainLayer> h((size_t)n);
  int aStride = 0, bStride = 0;
  for(int i = 0; i < n; i++) {
    const ConvTcPlan* p = members[i].plan;
    const Epilogue& ep = members[i].ep;
    const int act = ep.outAct ? ep.act : KB_ACT_IDENTITY;
    // layers without an activated output run any variant; the others must agree
    if(ep.outAct && c->act == KB_ACT_IDENTITY) c->act = act;
    if(!convChainEligible(p, ep) || p->dt != c->dt || p->BN != p0->BN || (ep.outAct && act != c->act)) { delete c; return nullptr; }
    ChainLayer& L = h[(size_t)i];
    std::memset(&L, 0, sizeof(L));
    L.tmA = p->tmA; L.tmB = p->tmB; L.tmRes = p->tmRes; L.tmRaw = p->tmRaw; L.tmAct = p->tmAct;
    ConvTcArgs& a = L.a;
    a.ep = ep;
    a.inC = p->inC; a.outC = p->outC; a.kY = p->kY; a.kX = p->kX;
    a.BN = p->BN; a.kChunks = p->kChunks; a.haloPad = p->haloPad; a.aRows = p->aRows;
    a.aSlotBytes = p->aRows * 128; a.bSlotBytes = p->BN * 128;
    a.idesc = p->idesc;
    a.tmaEpi = 1;
    a.doneCtr = (i + 1 < n) ? members[i].done : nullptr;
    a.depCtr = (i > 0) ? members[i - 1].done : nullptr;
    a.depTarget = (i > 0) ? (uint32_t)((members[i - 1].plan->outC / members[i - 1].plan->BN) * tcEpiWarps(TC_EPI_CG)) : 0u;
    if((i + 1 < n && !members[i].done)) { delete c; return nullptr; }
    // timing experiments only (results are wrong): 1 = no tile waits, 2 = no waits and no reports
    if(const char* e = getenv("KB_CHAIN_DEBUG")) {
      const int v = atoi(e);
      if(v >= 1) a.depCtr = nullptr;
      if(v >= 2) a.doneCtr = nullptr;
    }
    aStride = std::max(aStride, (a.aSlotBytes + 1023) / 1024 * 1024);
    bStride = std::max(bStride, (a.bSlotBytes + 1023) / 1024 * 1024);
    c->maxNTiles = std::max(c->maxNTiles, p->outC / p->BN);
  }
  ChainCfg& cfg = c->cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.numLayers = n;
  cfg.numA = 2;
  if(const char* e = getenv("KB_CHAIN_NUMA")) { int v = atoi(e); if(v >= 2 && v <= 4) cfg.numA = v; }
  cfg.aSlotStride = aStride;
  cfg.bSlotStride = bStride;
  cfg.epiWarpBytes = 3 * TC_UNIT_BYTES;  // two residual/raw units and one for the activated output
  const int fixed = (int)(CHAIN_MAX_LAYERS * sizeof(ConvTcArgs)) + 96 * 8 + 64 + 1024;
  const int budget = 227 * 1024 - fixed - tcEpiWarps(TC_EPI_CG) * cfg.epiWarpBytes - cfg.numA * aStride;
  int numB = budget / bStride;
  if(numB > 12) numB = 12;
  if(numB < 2) { delete c; return nullptr; }
  cfg.numB = numB;
  c->smemBytes = (size_t)cfg.numA * aStride + (size_t)numB * bStride + (size_t)tcEpiWarps(TC_EPI_CG) * cfg.epiWarpBytes + (size_t)fixed;
  cfg.tmemCols = 32;
  while((int)cfg.tmemCols < 2 * p0->BN) cfg.tmemCols *= 2;
  if(cudaMalloc(&c->dLayers, sizeof(ChainLayer) * (size_t)n) != cudaSuccess) { delete c; return nullptr; }
  if(cudaMemcpy(c->dLayers, h.data(), sizeof(ChainLayer) * (size_t)n, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(c->dLayers); delete c; return nullptr; }
  return c;
}

void convChainDestroy(ConvChainPlan* c) {
  if(!c) return;
  if(c->dLayers) cudaFree(c->dLayers);
  delete c;
}

cudaError_t launchConvChain(cudaStream_t st, const ConvChainPlan* c, Geom g, int* statusWord) {
  ChainCfg cfg = c->cfg;
  cfg.g = g;
  cfg.status = statusWord;
  cfg.tlSlot = 0;
#ifdef KB_TC_TRACE
  {
    const int idx = g_tlLaunch++;
    if(idx >= g_tlFirst && idx < g_tlFirst + TL_SLOTS) cfg.tlSlot = idx - g_tlFirst + 1;
  }
#endif
  // every CTA must be resident at the same time: one CTA per SM, never more CTAs than SMs
  const long long totalTiles = (long long)(g.rowsPad / TC_BM) * cfg.numLayers;
  const int grid = (int)std::min<long long>(totalTiles, (long long)c->numSMs);
  ConvChainKernelFn fn = c->dt == DT_F16 ? chainKernelForT<__half>(c->act) : chainKernelForT<__nv_bfloat16>(c->act);
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
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid); lc.blockDim = dim3(tcThreads(TC_EPI_CG, true)); lc.dynamicSmemBytes = c->smemBytes; lc.stream = st;
  cudaLaunchAttribute attr[1];
  int numAttrs = 0;
  if(usePdl) {
    attr[numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[numAttrs].val.programmaticStreamSerializationAllowed = 1;
    numAttrs++;
  }
  lc.attrs = attr; lc.numAttrs = numAttrs;
  return cudaLaunchKernelEx(&lc, fn, (const ChainLayer*)c->dLayers, cfg);
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded waits: a one-thread kernel waits, with the given limit, on a barrier that nothing ever arrives
// at.  The wait gives up, the kernel records its code in the status word exactly as the convolution kernels do on a
// time-out, and returns; the context stays usable.

enum { TC_ERR_SELFTEST_TIMEOUT = 199 };

__global__ void waitTimeoutSelfTestKernel(int* status, unsigned long long limitNs) {
  __shared__ uint64_t bar;
  __shared__ int abortFlag;
  if(threadIdx.x == 0) {
    abortFlag = 0;
    mbarInit(smemU32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool arrived = mbarWait(smemU32(&bar), 0u, &abortFlag, (uint64_t)limitNs);
    if(!arrived) atomicCAS(status, 0, TC_ERR_SELFTEST_TIMEOUT);
  }
}

cudaError_t launchWaitTimeoutSelfTest(cudaStream_t st, int* statusWord, unsigned long long limitNs) {
  if(limitNs > 1000000000ull) return cudaErrorInvalidValue;  // a self-test never waits longer than a second
  waitTimeoutSelfTestKernel<<<1, 32, 0, st>>>(statusWord, limitNs);
  return cudaGetLastError();
}

}  // namespace kb

#ifdef KB_TC_TRACE
extern "C" int kb_debug_trace(long long* out, int n) { return (int)cudaMemcpyFromSymbol(out, kb::g_tcTrace, sizeof(long long) * n); }
// Records the launches number first .. first + 11 (counted over tensor-core convolution launches from this call on).
extern "C" void kb_debug_timeline_arm(int first) { kb::g_tlLaunch = 0; kb::g_tlFirst = first; }
extern "C" int kb_debug_timeline(unsigned long long* out, int n) { return (int)cudaMemcpyFromSymbol(out, kb::g_tcTimeline, sizeof(unsigned long long) * n); }
#endif
