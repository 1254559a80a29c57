// Attention over the points of one board on sm_100a tensor cores (tcgen05), for head dimension 64.
//
// The tokens of a board are its padded rows (row = y*RW + x, kb_kernels.cuh): contiguous in memory, so Q, K and V
// tiles are plain 2-D TMA boxes of the QKV matrix; padding rows and off-board points are excluded as keys by an
// additive bias of -1e30 and produce zero output as queries (eigenbackend.cpp:1505-1536).  All keys of a board
// (<= 384 rows) are processed in one pass per 128-query tile:
//   S = Q K^T      MMAs into 384 TMEM columns (fp32)
//   softmax        two warps per query-row quarter, each over half of the keys: a pass for the maximum and a pass for
//                  exp and sum straight out of TMEM (the next 32-key chunk is in flight while one is processed);
//                  P is written in the activation dtype into shared memory in the K-major swizzled operand layout
//   O = P V        24 MMAs 128x64x16; V is used as it lies in memory (dv contiguous = MN-major B operand)
//   out = O / sum  read from TMEM, written with 16-byte stores
// Two kernels with the same arithmetic (identical bits):
//   attentionTcKernel    one CTA per (board, head) that runs the phases one after the other; it can rotate Q and K
//                        (rotary embedding) in place in shared memory first, for callers whose projection did not
//   attentionPipeKernel  persistent CTAs, a dedicated warp for TMA and MMA issue, two O buffers: the tensor core works
//                        on the neighbouring units while the softmax warps work on this one (see there)
// Waits are bounded as in the convolution kernel; on a time-out the status word is set and the CTA runs through its
// remaining barriers without touching data.
#include "kb_kernels.cuh"
#include "kb_tc_ptx.cuh"
#include "kb_act.cuh"

#include <mutex>

namespace kb {

constexpr int AT_SK = 384;     // keys per board handled in one pass (19x19: 19*20 = 380 rows)
constexpr int AT_D = 64;       // head dimension (q, k and v)
constexpr int AT_THREADS = 256;
constexpr int AT_TILE_BYTES = 128 * 128;  // 128 rows x 64 elements x 2 bytes
constexpr int AT_REL_MAX = 1536;          // floats of one head's relative-position table: (2Y-1)(2X-1) < 4*Y*X <= 4*AT_SK

enum { AT_ERR_TIMEOUT = 201 };

// Optional timeline instrumentation (build with -DKB_TC_TRACE): thread 0 of CTA 0 records SM cycle counts.
#ifdef KB_TC_TRACE
__device__ long long g_atTrace[256];
#define AT_TRACE(slot) do { if(blockIdx.x == 0 && threadIdx.x == 0) g_atTrace[(slot)] = clock64(); } while(0)
// threads 0, 32 and 160 (warps 0, 1 and 5) of CTA 0, while `cond` holds: 48 slots each from slot 64
#define AT_TRACE_W(cond, slot) do { if(blockIdx.x == 0 && (cond) && (threadIdx.x == 0 || threadIdx.x == 32 || threadIdx.x == 160)) \
  g_atTrace[64 + (threadIdx.x == 0 ? 0 : (threadIdx.x == 32 ? 48 : 96)) + (slot)] = clock64(); } while(0)
// the issuing thread of CTA 0: slots from 208
#define AT_TRACE_I(cond, slot) do { if(blockIdx.x == 0 && (cond)) g_atTrace[208 + (slot)] = clock64(); } while(0)
#else
#define AT_TRACE(slot) do { } while(0)
#define AT_TRACE_W(cond, slot) do { } while(0)
#define AT_TRACE_I(cond, slot) do { } while(0)
#endif

struct AttnTcArgs {
  Geom g;
  int heads, kvHeads;
  int qOff, kOff, vOff;   // column offsets of Q, K, V in the QKV matrix
  int keysValid;          // Y * RW: rows of a board that can hold keys
  const float* mask;
  void* out;
  int outStride;
  uint32_t idescS, idescS256, idescO;   // S = Q K^T for 128 keys, for 256 keys (the pipelined kernel), O = P V
  float scaleLog2e;       // 1/sqrt(dq) * log2(e)
  // Rotary tables in factored form, or NULL (Q and K are used as stored): the angle of pair p at point (x,y) is the sum
  // of an x part and a y part; ropeX [tableHeads][AT_D/2][X] and ropeY [tableHeads][AT_D/2][Y] hold (cos, sin) of the
  // parts.  A head's tables are a few KB, so they stay in L1.
  const float2* ropeX;
  const float2* ropeY;
  int tableHeads;
  const float* relBias;   // learned relative-position bias [heads][2*relY-1][2*relX-1] (BIAS kernels only)
  int relY, relX;
  int* status;
};

template <typename T> struct AtPack;
template <> struct AtPack<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
};
template <> struct AtPack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
};

template <typename T> struct AtUnpack;
template <> struct AtUnpack<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
};
template <> struct AtUnpack<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
};

// Rotary embedding (eigenbackend.cpp:1415-1451) applied in place to one 128-row x 64-channel tile that TMA put into
// shared memory with the 128-byte swizzle: channel pair (2p, 2p+1) of the row at board point (x,y) is rotated by the
// angle ax(p,x) + ay(p,y); cosine and sine of the sum come from the tabulated cosines and sines of the two parts.
// Rows that are not board points are left alone (they are masked out of the softmax, and their outputs are written as
// zeros).  The 16-byte shared-memory accesses of a quarter warp fall into distinct banks.
static_assert(AT_THREADS == 256, "ropeTileInPlace maps 256 threads onto 128 rows x 2 chunk phases");
template <typename T>
__device__ __forceinline__ void ropeTileInPlace(
  uint8_t* tile, int firstRow, int tableHead, const float2* __restrict__ ropeX, const float2* __restrict__ ropeY, const Geom& g, int tid) {
  // thread -> one row and every second 16-byte chunk of it (4 chunks = 16 channel pairs); all table values are
  // requested before any is used
  const int row = tid & 127, c0 = tid >> 7;
  const int br = firstRow + row;  // row inside the board's padded block
  const int y = br / g.RW, x = br - y * g.RW;
  if(y >= g.Y || x >= g.X) return;
  float2 ax[16], ay[16];
#pragma unroll
  for(int kk = 0; kk < 4; kk++) {
    const int p0 = tableHead * (AT_D / 2) + (c0 + 2 * kk) * 4;
#pragma unroll
    for(int k = 0; k < 4; k++) { ax[4 * kk + k] = __ldg(ropeX + (size_t)(p0 + k) * g.X + x); ay[4 * kk + k] = __ldg(ropeY + (size_t)(p0 + k) * g.Y + y); }
  }
#pragma unroll
  for(int kk = 0; kk < 4; kk++) {
    const int chunk = c0 + 2 * kk;
    uint4* p = reinterpret_cast<uint4*>(tile + row * 128 + ((chunk ^ (row & 7)) << 4));
    const uint4 val = *p;
    uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
    for(int k = 0; k < 4; k++) {
      const float2 a = ax[4 * kk + k], b = ay[4 * kk + k];
      const float cs = a.x * b.x - a.y * b.y, sn = a.y * b.x + a.x * b.y;
      const float2 v = AtUnpack<T>::unpack(w[k]);
      w[k] = AtPack<T>::pack(v.x * cs - v.y * sn, v.x * sn + v.y * cs);
    }
    *p = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

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

template <typename T, bool BIAS>
__global__ void __launch_bounds__(AT_THREADS, 1) attentionTcKernel(const __grid_constant__ CUtensorMap tmQKV, const AttnTcArgs a) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                         // 16 KiB
  uint8_t* sK = sQ + AT_TILE_BYTES;           // 3 x 16 KiB (128 keys each)
  uint8_t* sV = sK + 3 * AT_TILE_BYTES;       // 3 x 16 KiB
  uint8_t* sP = sV + 3 * AT_TILE_BYTES;       // 6 x 16 KiB (64 keys each), K-major operand layout
  float* sKb = reinterpret_cast<float*>(sP + 6 * AT_TILE_BYTES);  // [AT_SK] additive key bias: 0 on the board, -1e30 elsewhere
  float* sRed = sKb + AT_SK;                                      // [2][128] partial row maxima, then partial row sums
  // BIAS only: this head's bias table times log2(e), and for every key row its offset into it (ky * (2*relX-1) + kx)
  float* sRel = sRed + 256;                                       // [AT_REL_MAX]
  int* sKeyOff = reinterpret_cast<int*>(sRel + (BIAS ? AT_REL_MAX : 0));  // [AT_SK]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKeyOff + (BIAS ? AT_SK : 0));  // k (all tiles), q, mma1, mma2, v
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 5);
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
    for(int i = 0; i < 5; i++) mbarInit(smemU32(&bars[i]), 1);
    *abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 0) { tmemAlloc(smemU32(tmemSlot), 512); tmemRelinquish(); }
  for(int j = tid; j < AT_SK; j += AT_THREADS) sKb[j] = (j < a.keysValid && a.mask[boardRow + j] != 0.0f) ? 0.0f : -1e30f;
  if(BIAS) {
    const int W = 2 * a.relX - 1, relN = (2 * a.relY - 1) * W;
    for(int j = tid; j < relN; j += AT_THREADS) sRel[j] = a.relBias[(size_t)h * relN + j] * 1.4426950408889634f;
    for(int j = tid; j < AT_SK; j += AT_THREADS) {
      const int ky = j / a.g.RW, kx = j - ky * a.g.RW;
      sKeyOff[j] = (ky < a.g.Y && kx < a.g.X) ? ky * W + kx : 0;  // keys off the board: any valid entry, their key bias is -1e30
    }
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const uint32_t tmemS = tmemBase, tmemO = tmemBase + AT_SK;

  if(tid == 0) {
    // K and V of this (board, kv head) are loaded once and serve every query tile; the first Q tile rides along
    // K and Q first (S = Q K^T needs only them), V on a barrier of its own: it is not needed before O = P V
    mbarExpectTx(smemU32(&bars[0]), 3u * AT_TILE_BYTES);
    for(int j = 0; j < 3; j++) tmaLoad2d(smemU32(sK + j * AT_TILE_BYTES), &tmQKV, a.kOff + kvh * AT_D, boardRow + j * 128, smemU32(&bars[0]));
    mbarExpectTx(smemU32(&bars[1]), (uint32_t)AT_TILE_BYTES);
    tmaLoad2d(smemU32(sQ), &tmQKV, a.qOff + h * AT_D, boardRow, smemU32(&bars[1]));
    mbarExpectTx(smemU32(&bars[4]), 3u * AT_TILE_BYTES);
    for(int j = 0; j < 3; j++) tmaLoad2d(smemU32(sV + j * AT_TILE_BYTES), &tmQKV, a.vOff + kvh * AT_D, boardRow + j * 128, smemU32(&bars[4]));
  }

  // Shared-memory descriptors as 32-bit low words (start address, leading offset) plus the common high word, so that the
  // issuing thread spends an add per MMA
  const uint32_t descHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);  // stride offset | version | SWIZZLE_128B
  auto descLo = [](uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); };

  // Rotates Q of tile qt (and K, for the first tile) in shared memory if asked to, then has thread 0 issue S = Q K^T.
  auto issueScores = [&](int qt) {
    const uint32_t ph = (uint32_t)qt & 1u;
    bool landed = true;
    if(a.ropeX) {
      // every thread waits for the tiles and rotates its share; the rotated operands are made visible to the tensor core
      landed = (qt > 0 || mbarWait(smemU32(&bars[0]), 0u, abortFlag)) && mbarWait(smemU32(&bars[1]), ph, abortFlag);
      if(landed) {
        if(qt == 0) {
          const int thK = kvh * a.tableHeads / a.kvHeads;
          for(int j = 0; j < 3; j++) ropeTileInPlace<T>(sK + j * AT_TILE_BYTES, j * 128, thK, a.ropeX, a.ropeY, a.g, tid);
        }
        ropeTileInPlace<T>(sQ, qt * 128, h * a.tableHeads / a.heads, a.ropeX, a.ropeY, a.g, tid);
      }
      fenceProxyAsync();
      __syncthreads();
    }
    AT_TRACE(2 + qt * 8);
    if(tid == 0) {
      bool ok = landed && (qt > 0 || mbarWait(smemU32(&bars[0]), 0u, abortFlag)) && mbarWait(smemU32(&bars[1]), ph, abortFlag);
      if(ok) {
        tcFenceAfter();
        const uint32_t qLo = descLo(smemU32(sQ));
        for(int j = 0; j < 3; j++) {
          const uint32_t kLo = descLo(smemU32(sK + j * AT_TILE_BYTES));
#pragma unroll
          for(int k = 0; k < AT_D / 16; k++) ummaLoHi(tmemS + (uint32_t)(j * 128), qLo + 2 * k, kLo + 2 * k, descHi, a.idescS, k > 0 ? 1u : 0u);
        }
        ummaCommit(smemU32(&bars[2]));
      }
      else if(!*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, AT_ERR_TIMEOUT); }
    }
  };

  AT_TRACE(0);
  issueScores(0);
  for(int qt = 0; qt < numQTiles; qt++) {
    AT_TRACE(1 + qt * 8);
    const uint32_t ph = (uint32_t)qt & 1u;
    const int q0 = qt * 128;
    // ---- softmax: two warps per query row quarter, each over half of the keys ----
    const float qMask = (q0 + row < a.keysValid) ? a.mask[boardRow + q0 + row] : 0.0f;
    // this query's origin in the bias table (queries that are not board points produce zeros anyway and skip the bias)
    const float* qRel = nullptr;
    if(BIAS) {
      const int qr = q0 + row, qy = qr / a.g.RW, qx = qr - qy * a.g.RW;
      if(qy < a.g.Y && qx < a.g.X) qRel = sRel + (a.relY - 1 - qy) * (2 * a.relX - 1) + (a.relX - 1 - qx);
    }
    const int4* ko4 = reinterpret_cast<const int4*>(sKeyOff + half * (AT_SK / 2));
    bool ok = mbarWait(smemU32(&bars[2]), ph, abortFlag);
    if(!ok && !*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, AT_ERR_TIMEOUT); }
    if(tid == 0 && ok && qt + 1 < numQTiles) {
      // S = Q K^T has completed, so the Q tile is free: fetch the next one behind the softmax
      mbarExpectTx(smemU32(&bars[1]), (uint32_t)AT_TILE_BYTES);
      tmaLoad2d(smemU32(sQ), &tmQKV, a.qOff + h * AT_D, boardRow + q0 + 128, smemU32(&bars[1]));
    }
    AT_TRACE(3 + qt * 8);
    // Scores leave TMEM in chunks of 32 keys; the load of the next chunk is in flight while this one is processed.
    // Keys off the board carry a bias of -1e30, so they lose every maximum and their exponential is 0.
    constexpr int NCH = AT_SK / 2 / 32;
    const int cBegin = half * (AT_SK / 2);
    const uint32_t tS = tmemS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)cBegin;
    const float4* kb4 = reinterpret_cast<const float4*>(sKb + cBegin);
    float mx = -1e30f;
    if(ok) {
      tcFenceAfter();
      uint32_t r[2][32];
      float m4[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
      tmemLd32(tS, r[0]);
      tmemLdWaitFor(r[0]);
#pragma unroll
      for(int i = 0; i < NCH; i++) {
        if(i + 1 < NCH) tmemLd32(tS + (uint32_t)((i + 1) * 32), r[(i + 1) & 1]);
#pragma unroll
        for(int j = 0; j < 8; j++) {
          // everything in the base-2 exponent domain: t = score * scale * log2(e) + key bias (+ relative bias * log2(e))
          float4 b = kb4[i * 8 + j];
          if(BIAS && qRel) {
            const int4 ko = ko4[i * 8 + j];
            b.x += qRel[ko.x]; b.y += qRel[ko.y]; b.z += qRel[ko.z]; b.w += qRel[ko.w];
          }
          const float t0 = fmaf(__uint_as_float(r[i & 1][4 * j]), a.scaleLog2e, b.x), t1 = fmaf(__uint_as_float(r[i & 1][4 * j + 1]), a.scaleLog2e, b.y);
          const float t2 = fmaf(__uint_as_float(r[i & 1][4 * j + 2]), a.scaleLog2e, b.z), t3 = fmaf(__uint_as_float(r[i & 1][4 * j + 3]), a.scaleLog2e, b.w);
          m4[0] = fmaxf(m4[0], t0); m4[1] = fmaxf(m4[1], t1); m4[2] = fmaxf(m4[2], t2); m4[3] = fmaxf(m4[3], t3);
          if(BIAS) {
            r[i & 1][4 * j] = __float_as_uint(t0); r[i & 1][4 * j + 1] = __float_as_uint(t1);
            r[i & 1][4 * j + 2] = __float_as_uint(t2); r[i & 1][4 * j + 3] = __float_as_uint(t3);
          }
        }
        // with a relative-position bias the scaled and biased scores go back into TMEM, so that the second pass does
        // not gather the bias again
        if(BIAS) tmemSt32(tS + (uint32_t)(i * 32), r[i & 1]);
        if(i + 1 < NCH) tmemLdWaitFor(r[(i + 1) & 1]);
      }
      mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      if(BIAS) tmemStWait();
    }
    AT_TRACE(4 + qt * 8);
    sRed[half * 128 + row] = mx;
    __syncthreads();
    mx = fmaxf(sRed[row], sRed[128 + row]);
    __syncthreads();
    float sum = 0.0f;
    if(ok) {
      const int sw = row & 7;
      const float mxs = mx;  // the maximum is already in the exponent domain
      uint32_t r[2][32];
      float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      tmemLd32(tS, r[0]);
      tmemLdWaitFor(r[0]);
#pragma unroll
      for(int i = 0; i < NCH; i++) {
        if(i + 1 < NCH) tmemLd32(tS + (uint32_t)((i + 1) * 32), r[(i + 1) & 1]);
        const int c = cBegin + i * 32;
        // P chunk of 64 keys = one 128-byte swizzled row per query; this 32-key group is its half (c/32)&1
        uint8_t* pRow = sP + (size_t)(c / 64) * AT_TILE_BYTES + row * 128;
        const int halfSel = (c / 32) & 1;
#pragma unroll
        for(int jj = 0; jj < 4; jj++) {
          float p[8];
#pragma unroll
          for(int k = 0; k < 2; k++) {
            if(BIAS) {
              // the first pass left scale * score + bias in TMEM
              p[4 * k] = ex2Approx(__uint_as_float(r[i & 1][8 * jj + 4 * k]) - mxs);
              p[4 * k + 1] = ex2Approx(__uint_as_float(r[i & 1][8 * jj + 4 * k + 1]) - mxs);
              p[4 * k + 2] = ex2Approx(__uint_as_float(r[i & 1][8 * jj + 4 * k + 2]) - mxs);
              p[4 * k + 3] = ex2Approx(__uint_as_float(r[i & 1][8 * jj + 4 * k + 3]) - mxs);
            }
            else {
              const float4 b = kb4[i * 8 + 2 * jj + k];
              p[4 * k] = ex2Approx(fmaf(__uint_as_float(r[i & 1][8 * jj + 4 * k]), a.scaleLog2e, b.x - mxs));
              p[4 * k + 1] = ex2Approx(fmaf(__uint_as_float(r[i & 1][8 * jj + 4 * k + 1]), a.scaleLog2e, b.y - mxs));
              p[4 * k + 2] = ex2Approx(fmaf(__uint_as_float(r[i & 1][8 * jj + 4 * k + 2]), a.scaleLog2e, b.z - mxs));
              p[4 * k + 3] = ex2Approx(fmaf(__uint_as_float(r[i & 1][8 * jj + 4 * k + 3]), a.scaleLog2e, b.w - mxs));
            }
            s4[0] += p[4 * k]; s4[1] += p[4 * k + 1]; s4[2] += p[4 * k + 2]; s4[3] += p[4 * k + 3];
          }
          uint4 o;
          o.x = AtPack<T>::pack(p[0], p[1]); o.y = AtPack<T>::pack(p[2], p[3]);
          o.z = AtPack<T>::pack(p[4], p[5]); o.w = AtPack<T>::pack(p[6], p[7]);
          *reinterpret_cast<uint4*>(pRow + (((halfSel * 4 + jj) ^ sw) << 4)) = o;
        }
        if(i + 1 < NCH) tmemLdWaitFor(r[(i + 1) & 1]);
      }
      sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
    }
    AT_TRACE(5 + qt * 8);
    sRed[half * 128 + row] = sum;
    fenceProxyAsync();
    tcFenceBefore();
    __syncthreads();
    const float rowSum = sRed[row] + sRed[128 + row];
    if(tid == 0 && !*abortFlag && (qt > 0 || mbarWait(smemU32(&bars[4]), 0u, abortFlag))) {
      tcFenceAfter();
      uint32_t acc = 0;
      for(int kc = 0; kc < AT_SK / 64; kc++) {
        const uint32_t pLo = descLo(smemU32(sP + (size_t)kc * AT_TILE_BYTES));          // 64 keys of P: one swizzle atom per row
        const uint32_t vLo = descLo(smemU32(sV) + (uint32_t)(kc * 64) * 128u);         // the same 64 key rows of V
#pragma unroll
        for(int k = 0; k < 4; k++) {
          // 16 keys further: 32 bytes along K inside P's atom, 16 rows (2048 bytes) down in V
          ummaLoHi(tmemO, pLo + 2 * k, vLo + (uint32_t)k * 128u, descHi, a.idescO, acc);
          acc = 1;
        }
      }
      ummaCommit(smemU32(&bars[3]));
    }
    // S of this tile has been consumed and its MMAs for O are queued: rotate the next Q tile and queue its S = Q K^T
    // behind them, so that both run while the threads read O out
    if(qt + 1 < numQTiles) issueScores(qt + 1);
    AT_TRACE(6 + qt * 8);
    ok = !*abortFlag && mbarWait(smemU32(&bars[3]), ph, abortFlag);
    AT_TRACE(7 + qt * 8);
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
    AT_TRACE(8 + qt * 8);
    // No barrier here: the next tile's P is written only after this wait on the O barrier, and its O MMAs are issued
    // behind the softmax barriers, which every thread reaches after it has read this tile's O.
  }
  tcFenceBefore();
  __syncthreads();
  if(warp == 0) { tcFenceAfter(); tmemDealloc(tmemBase, 512); }
}

// ---------------------------------------------------------------------------------------------
// Pipelined variant, used when Q and K arrive already rotated (the projection's epilogue applied the rotary embedding)
// or the block has no rotary embedding.  Same arithmetic as attentionTcKernel, instruction for instruction, so the two
// produce identical bits; what differs is who does what when:
//   * persistent CTAs: the (board, head, query tile) units are split into equal contiguous ranges, one per CTA, so all
//     SMs finish together; K and V of a (board, kv head) stay in shared memory while consecutive units use them, and
//     the next unit's Q (and K) are fetched as soon as the MMAs that read the buffers have completed;
//   * a ninth warp issues every TMA load and every MMA (its warpgroup hands most of its registers to the softmax
//     warpgroups, whose two passes want more than an even split of the register file gives them); the eight softmax
//     warps never issue one and never meet it at a CTA-wide barrier (they synchronise among themselves on named
//     barrier 1 and with the issuer through mbarriers);
//   * O has two TMEM buffers, so a unit's output is read out of TMEM one unit later, after the second softmax pass of
//     the next unit, while the tensor core computes the S = Q K^T after that; O = P V of unit i runs behind S of unit
//     i+1, under unit i+1's softmax passes, and releases P to the second pass chunk by chunk (64 keys at a time).
// Order on the tensor core: S(0), S(1), PV(0), S(2), PV(1), ...  S(i+1) is issued when every softmax warp has left the
// second pass of unit i (S consumed, P complete).  Per unit a softmax warp: wait S | pass 1 (maximum) | pass 2 (exp,
// P, sum) | signal | row sums | read out O of the unit before.
constexpr int AP_THREADS = 384;  // two warpgroups of softmax warps and the issuer's warpgroup (one of its warps works)
enum {
  AP_K_FULL = 0, AP_V_FULL, AP_Q_FULL, AP_S_FULL, AP_SM_DONE, AP_O_FULL, AP_O_FREE = AP_O_FULL + 2,
  AP_P_FREE = AP_O_FREE + 2,                // one per 64-key chunk of P: O = P V of the unit before has read it
  AP_NUM_BARS = AP_P_FREE + AT_SK / 64
};

__device__ __forceinline__ void softmaxWarpsSync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <typename T, bool BIAS>
__global__ void __launch_bounds__(AP_THREADS, 1) attentionPipeKernel(const __grid_constant__ CUtensorMap tmQKV, const AttnTcArgs a) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                         // 16 KiB
  uint8_t* sK = sQ + AT_TILE_BYTES;           // 3 x 16 KiB (128 keys each)
  uint8_t* sV = sK + 3 * AT_TILE_BYTES;       // 3 x 16 KiB
  uint8_t* sP = sV + 3 * AT_TILE_BYTES;       // 6 x 16 KiB (64 keys each), K-major operand layout
  float* sKb = reinterpret_cast<float*>(sP + 6 * AT_TILE_BYTES);  // [AT_SK] additive key bias: 0 on the board, -1e30 elsewhere
  float* sMax = sKb + AT_SK;                                      // [2][128] partial row maxima
  float* sSum = sMax + 256;                                       // [2][128] partial row sums
  float* sRel = sSum + 256;                                       // [AT_REL_MAX] (BIAS) this head's bias table times log2(e)
  int* sKeyOff = reinterpret_cast<int*>(sRel + (BIAS ? AT_REL_MAX : 0));  // [AT_SK] (BIAS) offset of every key row into it
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKeyOff + (BIAS ? AT_SK : 0));
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + AP_NUM_BARS);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  AT_TRACE(0);
  if(tid == 0) {
    for(int i = 0; i < AP_NUM_BARS; i++) mbarInit(smemU32(&bars[i]), (i == AP_SM_DONE || (i >= AP_O_FREE && i < AP_P_FREE)) ? 8 : 1);
    *abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if(warp == 0) { tmemAlloc(smemU32(tmemSlot), 512); tmemRelinquish(); }
  if(BIAS) {
    const int W = 2 * a.relX - 1;
    for(int j = tid; j < AT_SK; j += AP_THREADS) {
      const int ky = j / a.g.RW, kx = j - ky * a.g.RW;
      sKeyOff[j] = (ky < a.g.Y && kx < a.g.X) ? ky * W + kx : 0;  // keys off the board: any valid entry, their key bias is -1e30
    }
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const uint32_t tmemS = tmemBase, tmemO = tmemBase + AT_SK;  // O buffer b at tmemO + 64 b

  // this CTA's units: unit u = (item, query tile), item = (board, head)
  const int numQTiles = (a.keysValid + 127) / 128;
  const int units = a.g.n * a.heads * numQTiles;
  const int u0 = (int)((long long)blockIdx.x * units / gridDim.x), u1 = (int)((long long)(blockIdx.x + 1) * units / gridDim.x);
  const int headsPerKv = a.heads / a.kvHeads;
  auto giveUp = [&]() { if(!*abortFlag) { *abortFlag = 1; atomicCAS(a.status, 0, AT_ERR_TIMEOUT); } };

  if(warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if(warp == 8 && lane == 0 && u1 > u0) {
      // ---------------- issuer: every TMA load and every MMA ----------------
      const uint32_t descHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);  // stride offset | version | SWIZZLE_128B
      auto descLo = [](uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); };
      bool ok = true;
      uint32_t kWaited = 0, vWaited = 0, qWaited = 0;   // completed phases of the K, V and Q barriers this thread has consumed
      bool kPending = false, vPending = false, qPending = false;
      int kKey = -1, vKey = -1;            // (board, kv head) whose K / V is in shared memory or on its way
      auto decode = [&](int u, int& n, int& h, int& qt) {
        const int item = u / numQTiles;
        qt = u - item * numQTiles; n = item / a.heads; h = item - n * a.heads;
      };
      auto loadK = [&](int n, int kvh) {
        mbarExpectTx(smemU32(&bars[AP_K_FULL]), 3u * AT_TILE_BYTES);
        for(int j = 0; j < 3; j++) tmaLoad2d(smemU32(sK + j * AT_TILE_BYTES), &tmQKV, a.kOff + kvh * AT_D, n * a.g.PB + j * 128, smemU32(&bars[AP_K_FULL]));
        kPending = true; kKey = n * a.kvHeads + kvh;
      };
      auto loadV = [&](int n, int kvh) {
        mbarExpectTx(smemU32(&bars[AP_V_FULL]), 3u * AT_TILE_BYTES);
        for(int j = 0; j < 3; j++) tmaLoad2d(smemU32(sV + j * AT_TILE_BYTES), &tmQKV, a.vOff + kvh * AT_D, n * a.g.PB + j * 128, smemU32(&bars[AP_V_FULL]));
        vPending = true; vKey = n * a.kvHeads + kvh;
      };
      auto loadQ = [&](int n, int h, int qt) {
        mbarExpectTx(smemU32(&bars[AP_Q_FULL]), (uint32_t)AT_TILE_BYTES);
        tmaLoad2d(smemU32(sQ), &tmQKV, a.qOff + h * AT_D, n * a.g.PB + qt * 128, smemU32(&bars[AP_Q_FULL]));
        qPending = true;
      };
      // O = P V of the unit with local index j (every softmax warp has left its second pass)
      auto issuePV = [&](int j) {
        const int b = j & 1;
        if(ok && vPending) {
          if(mbarWait(smemU32(&bars[AP_V_FULL]), vWaited & 1u, abortFlag)) { vWaited++; vPending = false; }
          else ok = false;
        }
        // the softmax warps have read this O buffer's previous contents (unit j-2) out of TMEM
        ok = ok && mbarWait(smemU32(&bars[AP_O_FREE + b]), (((uint32_t)j >> 1) & 1u) ^ 1u, abortFlag);
        if(!ok) return;
        tcFenceAfter();
        uint32_t acc = 0;
        for(int kc = 0; kc < AT_SK / 64; kc++) {
          const uint32_t pLo = descLo(smemU32(sP + (size_t)kc * AT_TILE_BYTES));   // 64 keys of P: one swizzle atom per row
          const uint32_t vLo = descLo(smemU32(sV) + (uint32_t)(kc * 64) * 128u);  // the same 64 key rows of V
#pragma unroll
          for(int k = 0; k < 4; k++) {
            // 16 keys further: 32 bytes along K inside P's atom, 16 rows (2048 bytes) down in V
            ummaLoHi(tmemO + (uint32_t)(b * AT_D), pLo + 2 * k, vLo + (uint32_t)k * 128u, descHi, a.idescO, acc);
            acc = 1;
          }
          ummaCommit(smemU32(&bars[AP_P_FREE + kc]));  // this chunk of P may be overwritten by the next unit's second pass
        }
        ummaCommit(smemU32(&bars[AP_O_FULL + b]));
      };
      {
        int n, h, qt;
        decode(u0, n, h, qt);
        loadK(n, h / headsPerKv);
        loadQ(n, h, qt);
        loadV(n, h / headsPerKv);
      }
      for(int u = u0; u < u1; u++) {
        const int i = u - u0;
        int n, h, qt;
        decode(u, n, h, qt);
        const int key = n * a.kvHeads + h / headsPerKv;
        // operands of S(i)
        if(ok && mbarWait(smemU32(&bars[AP_Q_FULL]), qWaited & 1u, abortFlag)) { qWaited++; qPending = false; }
        else ok = false;
        if(ok && kPending) {
          if(mbarWait(smemU32(&bars[AP_K_FULL]), kWaited & 1u, abortFlag)) { kWaited++; kPending = false; }
          else ok = false;
        }
        // S of the unit before has been consumed and its P is complete
        if(i > 0) ok = ok && mbarWait(smemU32(&bars[AP_SM_DONE]), (uint32_t)(i - 1) & 1u, abortFlag);
        AT_TRACE_I(i < 6, i * 8 + 0);
        if(ok) {
          tcFenceAfter();
          // the three key tiles lie back to back in the operand layout (8-key groups 1024 bytes apart throughout), so
          // the first two go through one 256-wide MMA per 16 channels: an MMA's cost is mostly fixed (8 instead of 12)
          const uint32_t qLo = descLo(smemU32(sQ));
          const uint32_t kLo0 = descLo(smemU32(sK)), kLo2 = descLo(smemU32(sK + 2 * AT_TILE_BYTES));
#pragma unroll
          for(int k = 0; k < AT_D / 16; k++) ummaLoHi(tmemS, qLo + 2 * k, kLo0 + 2 * k, descHi, a.idescS256, k > 0 ? 1u : 0u);
#pragma unroll
          for(int k = 0; k < AT_D / 16; k++) ummaLoHi(tmemS + 256u, qLo + 2 * k, kLo2 + 2 * k, descHi, a.idescS, k > 0 ? 1u : 0u);
          ummaCommit(smemU32(&bars[AP_S_FULL]));
        }
        AT_TRACE_I(i < 6, i * 8 + 1);
        if(i > 0) issuePV(i - 1);
        AT_TRACE_I(i < 6, i * 8 + 2);
        // S(i) has completed: the Q buffer (and K, if the next unit belongs to another board or kv head) is free
        ok = ok && mbarWait(smemU32(&bars[AP_S_FULL]), (uint32_t)i & 1u, abortFlag);
        AT_TRACE_I(i < 6, i * 8 + 3);
        if(ok && u + 1 < u1) {
          int n2, h2, qt2;
          decode(u + 1, n2, h2, qt2);
          loadQ(n2, h2, qt2);
          if(n2 * a.kvHeads + h2 / headsPerKv != kKey) loadK(n2, h2 / headsPerKv);
        }
        // V of this unit's (board, kv head), once O = P V of the unit before has read the old one
        if(ok && vKey != key) {
          if(i > 0) ok = ok && mbarWait(smemU32(&bars[AP_O_FULL + ((i - 1) & 1)]), (((uint32_t)(i - 1)) >> 1) & 1u, abortFlag);
          if(ok) loadV(n, h / headsPerKv);
        }
        if(!ok) break;
      }
      if(ok) {
        const int last = u1 - 1 - u0;
        ok = mbarWait(smemU32(&bars[AP_SM_DONE]), (uint32_t)last & 1u, abortFlag);
        if(ok) issuePV(last);
      }
      if(!ok) {
        giveUp();
        // loads that were requested and never consumed: give them (bounded) time to land before the CTA exits; these
        // waits must not return early because the CTA has given up, so they watch a flag that stays 0
        volatile int keepWaiting = 0;
        if(qPending) mbarWait(smemU32(&bars[AP_Q_FULL]), qWaited & 1u, &keepWaiting, 1000000ull);
        if(kPending) mbarWait(smemU32(&bars[AP_K_FULL]), kWaited & 1u, &keepWaiting, 1000000ull);
        if(vPending) mbarWait(smemU32(&bars[AP_V_FULL]), vWaited & 1u, &keepWaiting, 1000000ull);
      }
    }
  }
  else {
    // ---------------- softmax warps: two per TMEM lane quarter, each over half of the keys ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int half = warp >> 2;          // which half of the keys (softmax) / of the output columns this warp handles
    const int row = quarter * 32 + lane; // query row inside the tile
    constexpr int NCH = AT_SK / 2 / 32;
    const int cBegin = half * (AT_SK / 2);
    const uint32_t tS = tmemS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)cBegin;
    const float4* kb4 = reinterpret_cast<const float4*>(sKb + cBegin);
    const int4* ko4 = reinterpret_cast<const int4*>(sKeyOff + half * (AT_SK / 2));
    const float2 scale2 = make_float2(a.scaleLog2e, a.scaleLog2e);
    int curBoard = -1, curHead = -1;
    float invPrev = 0.0f;       // 1 / row sum of the unit whose O is still in TMEM
    T* outWarpPrev = nullptr;   // that unit: where row 0, column 0 of this warp's 32 rows x 32 output columns goes
    int rowsValidPrev = 0;      // that unit: how many of this warp's 32 rows lie inside the board's block of rows
    // Reads the O buffer of the unit with local index j out of TMEM and writes the normalised values.  A thread holds
    // its row's 32 values as four 16-byte pieces; groups of four lanes transpose them (piece c of the group's four rows
    // ends up in lane c), so that a store instruction covers eight whole 64-byte row segments instead of 32 scattered
    // 16-byte pieces.
    auto writeOut = [&](int j) {
      const int b = j & 1;
      AT_TRACE_W(j == 2, 12);
      bool ok = !*abortFlag && mbarWait(smemU32(&bars[AP_O_FULL + b]), ((uint32_t)j >> 1) & 1u, abortFlag);
      if(!ok) giveUp();
      AT_TRACE_W(j == 2, 13);
      if(ok) {
        tcFenceAfter();
        uint32_t r[32];
        tmemLd32(tmemO + (uint32_t)(b * AT_D) + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 32), r);
        tmemLdWait();
        AT_TRACE_W(j == 2, 14);
        const float inv = invPrev;
        uint4 v[4];
#pragma unroll
        for(int jj = 0; jj < 4; jj++) {
          v[jj].x = AtPack<T>::pack(__uint_as_float(r[8 * jj]) * inv, __uint_as_float(r[8 * jj + 1]) * inv);
          v[jj].y = AtPack<T>::pack(__uint_as_float(r[8 * jj + 2]) * inv, __uint_as_float(r[8 * jj + 3]) * inv);
          v[jj].z = AtPack<T>::pack(__uint_as_float(r[8 * jj + 4]) * inv, __uint_as_float(r[8 * jj + 5]) * inv);
          v[jj].w = AtPack<T>::pack(__uint_as_float(r[8 * jj + 6]) * inv, __uint_as_float(r[8 * jj + 7]) * inv);
        }
        auto xchg = [&](uint4& keepLo, uint4& keepHi, int bit) {
          // lanes with the bit clear keep keepLo and trade keepHi for the partner's keepLo; the others the reverse
          const bool hi = (lane & bit) != 0;
          uint4 send = hi ? keepLo : keepHi, got;
          got.x = __shfl_xor_sync(0xffffffffu, send.x, bit); got.y = __shfl_xor_sync(0xffffffffu, send.y, bit);
          got.z = __shfl_xor_sync(0xffffffffu, send.z, bit); got.w = __shfl_xor_sync(0xffffffffu, send.w, bit);
          if(hi) keepLo = got; else keepHi = got;
        };
        xchg(v[0], v[1], 1); xchg(v[2], v[3], 1);
        xchg(v[0], v[2], 2); xchg(v[1], v[3], 2);
        // now v[k] = piece (lane & 3) of the row of lane (lane & ~3) + k
        AT_TRACE_W(j == 2, 15);
        const int r0 = lane & ~3, c = lane & 3;
#pragma unroll
        for(int k = 0; k < 4; k++)
          if(r0 + k < rowsValidPrev) *reinterpret_cast<uint4*>(outWarpPrev + (size_t)(r0 + k) * a.outStride + c * 8) = v[k];
        AT_TRACE_W(j == 2, 16);
      }
      tcFenceBefore();
      __syncwarp();
      if(lane == 0) mbarArrive(smemU32(&bars[AP_O_FREE + b]));
      AT_TRACE_W(j == 2, 17);
    };
    for(int u = u0; u < u1; u++) {
      const int i = u - u0;
      const int item = u / numQTiles, qt = u - item * numQTiles, n = item / a.heads, h = item - n * a.heads;
      const int boardRow = n * a.g.PB, q0 = qt * 128;
      // per-board key mask and per-head bias table; every softmax warp has left the previous unit's second pass (the
      // row-sum exchange lies in between)
      const bool newBoard = n != curBoard, newHead = BIAS && h != curHead;
      if(newBoard) {
        for(int j = tid; j < AT_SK; j += 256) sKb[j] = (j < a.keysValid && a.mask[boardRow + j] != 0.0f) ? 0.0f : -1e30f;
        curBoard = n;
      }
      if(newHead) {
        const int relN = (2 * a.relY - 1) * (2 * a.relX - 1);
        for(int j = tid; j < relN; j += 256) sRel[j] = a.relBias[(size_t)h * relN + j] * 1.4426950408889634f;
        curHead = h;
      }
      if(newBoard || newHead) softmaxWarpsSync();
      const float qMask = (q0 + row < a.keysValid) ? a.mask[boardRow + q0 + row] : 0.0f;
      // this query's origin in the bias table (queries that are not board points produce zeros anyway and skip the bias)
      const float* qRel = nullptr;
      if(BIAS) {
        const int qr = q0 + row, qy = qr / a.g.RW, qx = qr - qy * a.g.RW;
        if(qy < a.g.Y && qx < a.g.X) qRel = sRel + (a.relY - 1 - qy) * (2 * a.relX - 1) + (a.relX - 1 - qx);
      }
      if(i < 7) AT_TRACE(1 + i * 8);
      bool ok = mbarWait(smemU32(&bars[AP_S_FULL]), (uint32_t)i & 1u, abortFlag);
      if(!ok) giveUp();
      if(i < 7) AT_TRACE(2 + i * 8);
      AT_TRACE_W(i == 3, 0);
      // Scores leave TMEM in chunks of 32 keys; the load of the next chunk is in flight while this one is processed.
      // Keys off the board carry a bias of -1e30, so they lose every maximum and their exponential is 0.
      float mx = -1e30f;
      if(ok) {
        tcFenceAfter();
        uint32_t r[2][32];
        float m4[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
        tmemLd32(tS, r[0]);
        tmemLdWaitFor(r[0]);
#pragma unroll
        for(int ii = 0; ii < NCH; ii++) {
          if(ii + 1 < NCH) tmemLd32(tS + (uint32_t)((ii + 1) * 32), r[(ii + 1) & 1]);
#pragma unroll
          for(int j = 0; j < 8; j++) {
            // everything in the base-2 exponent domain: t = score * scale * log2(e) + key bias (+ relative bias * log2(e))
            float4 b = kb4[ii * 8 + j];
            if(BIAS && qRel) {
              const int4 ko = ko4[ii * 8 + j];
              b.x += qRel[ko.x]; b.y += qRel[ko.y]; b.z += qRel[ko.z]; b.w += qRel[ko.w];
            }
            // packed fp32 (two IEEE fused multiply-adds per instruction: the same bits as the scalar form)
            const float2 t01 = __ffma2_rn(make_float2(__uint_as_float(r[ii & 1][4 * j]), __uint_as_float(r[ii & 1][4 * j + 1])), scale2, make_float2(b.x, b.y));
            const float2 t23 = __ffma2_rn(make_float2(__uint_as_float(r[ii & 1][4 * j + 2]), __uint_as_float(r[ii & 1][4 * j + 3])), scale2, make_float2(b.z, b.w));
            m4[0] = fmaxf(m4[0], t01.x); m4[1] = fmaxf(m4[1], t01.y);
            m4[2] = fmaxf(m4[2], t23.x); m4[3] = fmaxf(m4[3], t23.y);
            if(BIAS) {
              r[ii & 1][4 * j] = __float_as_uint(t01.x); r[ii & 1][4 * j + 1] = __float_as_uint(t01.y);
              r[ii & 1][4 * j + 2] = __float_as_uint(t23.x); r[ii & 1][4 * j + 3] = __float_as_uint(t23.y);
            }
          }
          // with a relative-position bias the scaled and biased scores go back into TMEM, so that the second pass
          // does not gather the bias again
          if(BIAS) tmemSt32(tS + (uint32_t)(ii * 32), r[ii & 1]);
          if(ii + 1 < NCH) tmemLdWaitFor(r[(ii + 1) & 1]);
          AT_TRACE_W(i == 3, 20 + ii);
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        if(BIAS) tmemStWait();
      }
      AT_TRACE_W(i == 3, 1);
      sMax[half * 128 + row] = mx;
      softmaxWarpsSync();
      AT_TRACE_W(i == 3, 2);
      mx = fmaxf(sMax[row], sMax[128 + row]);
      if(i < 7) AT_TRACE(3 + i * 8);
      if(i < 7) AT_TRACE(4 + i * 8);
      AT_TRACE_W(i == 3, 3);
      float sum = 0.0f;
      bool pOk = true;
      if(ok && !*abortFlag) {
        const int sw = row & 7;
        const float2 negMx2 = make_float2(-mx, -mx);  // the maximum is already in the exponent domain
        uint32_t r[2][32];
        float2 s2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};  // four running sums, as in the scalar form
        tmemLd32(tS, r[0]);
        tmemLdWaitFor(r[0]);
#pragma unroll
        for(int ii = 0; ii < NCH; ii++) {
          if(ii + 1 < NCH) tmemLd32(tS + (uint32_t)((ii + 1) * 32), r[(ii + 1) & 1]);
          const int c = cBegin + ii * 32;
          // O = P V of the unit before runs behind this unit's S = Q K^T and may still be reading P: a 64-key chunk is
          // written once the MMAs that read it have completed
          // (the MMAs read the chunks in order, so a chunk's barrier also covers the chunks before it: the warps of
          // the first half of the keys wait once, for their last chunk, which is free long before they start; those
          // of the second half wait for their first chunk and then for their last)
          if(i > 0 && (ii == 0 || (half == 1 && ii == 2)))
            pOk = mbarWait(smemU32(&bars[AP_P_FREE + (half == 0 ? 2 : (ii == 0 ? 3 : 5))]), (uint32_t)(i - 1) & 1u, abortFlag) && pOk;
          // P chunk of 64 keys = one 128-byte swizzled row per query; this 32-key group is its half (c/32)&1
          uint8_t* pRow = sP + (size_t)(c / 64) * AT_TILE_BYTES + row * 128;
          const int halfSel = (c / 32) & 1;
#pragma unroll
          for(int jj = 0; jj < 4; jj++) {
            float p[8];
#pragma unroll
            for(int k = 0; k < 2; k++) {
              float2 t01, t23;
              if(BIAS) {
                // the first pass left scale * score + bias in TMEM
                t01 = __fadd2_rn(make_float2(__uint_as_float(r[ii & 1][8 * jj + 4 * k]), __uint_as_float(r[ii & 1][8 * jj + 4 * k + 1])), negMx2);
                t23 = __fadd2_rn(make_float2(__uint_as_float(r[ii & 1][8 * jj + 4 * k + 2]), __uint_as_float(r[ii & 1][8 * jj + 4 * k + 3])), negMx2);
              }
              else {
                const float4 b = kb4[ii * 8 + 2 * jj + k];
                t01 = __ffma2_rn(make_float2(__uint_as_float(r[ii & 1][8 * jj + 4 * k]), __uint_as_float(r[ii & 1][8 * jj + 4 * k + 1])), scale2,
                                 __fadd2_rn(make_float2(b.x, b.y), negMx2));
                t23 = __ffma2_rn(make_float2(__uint_as_float(r[ii & 1][8 * jj + 4 * k + 2]), __uint_as_float(r[ii & 1][8 * jj + 4 * k + 3])), scale2,
                                 __fadd2_rn(make_float2(b.z, b.w), negMx2));
              }
              p[4 * k] = ex2Approx(t01.x); p[4 * k + 1] = ex2Approx(t01.y);
              p[4 * k + 2] = ex2Approx(t23.x); p[4 * k + 3] = ex2Approx(t23.y);
              s2[0] = __fadd2_rn(s2[0], make_float2(p[4 * k], p[4 * k + 1]));
              s2[1] = __fadd2_rn(s2[1], make_float2(p[4 * k + 2], p[4 * k + 3]));
            }
            uint4 o;
            o.x = AtPack<T>::pack(p[0], p[1]); o.y = AtPack<T>::pack(p[2], p[3]);
            o.z = AtPack<T>::pack(p[4], p[5]); o.w = AtPack<T>::pack(p[6], p[7]);
            *reinterpret_cast<uint4*>(pRow + (((halfSel * 4 + jj) ^ sw) << 4)) = o;
          }
          if(ii + 1 < NCH) tmemLdWaitFor(r[(ii + 1) & 1]);
          AT_TRACE_W(i == 3, 4 + ii);
        }
        sum = (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
      }
      if(!pOk) giveUp();
      // this warp has consumed its part of S and written its part of P
      fenceProxyAsync();
      tcFenceBefore();
      __syncwarp();
      if(lane == 0) mbarArrive(smemU32(&bars[AP_SM_DONE]));
      if(i < 7) AT_TRACE(5 + i * 8);
      AT_TRACE_W(i == 3, 10);
      sSum[half * 128 + row] = sum;
      softmaxWarpsSync();
      AT_TRACE_W(i == 3, 11);
      const float rowSum = sSum[row] + sSum[128 + row];
      // the unit before: its O = P V has long completed; reading it out now overlaps the next unit's S = Q K^T
      if(i > 0) writeOut(i - 1);
      invPrev = (qMask != 0.0f && rowSum > 0.0f) ? 1.0f / rowSum : 0.0f;
      outWarpPrev = reinterpret_cast<T*>(a.out) + (size_t)(boardRow + q0 + quarter * 32) * a.outStride + h * AT_D + half * 32;
      rowsValidPrev = a.g.PB - (q0 + quarter * 32);
    }
    if(u1 > u0) writeOut(u1 - 1 - u0);
    AT_TRACE(60);
  }
  tcFenceBefore();
  __syncthreads();
  if(warp == 0) { tcFenceAfter(); tmemDealloc(tmemBase, 512); }
}

// ---------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFnA)(
  CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct AttnTcPlan {
  CUtensorMap tmQKV;
  int dt;
  size_t smemBytes;      // attentionTcKernel
  size_t smemBytesPipe;  // attentionPipeKernel
  int numSMs;
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
  p->smemBytes = 13 * (size_t)AT_TILE_BYTES + (AT_SK + 256 + AT_REL_MAX + AT_SK) * sizeof(float) + 5 * 8 + 16 + 1024;
  cudaError_t e1 = cudaFuncSetAttribute(attentionTcKernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smemBytes);
  cudaError_t e2 = cudaFuncSetAttribute(attentionTcKernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smemBytes);
  if(e1 == cudaSuccess) e1 = cudaFuncSetAttribute(attentionTcKernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smemBytes);
  if(e2 == cudaSuccess) e2 = cudaFuncSetAttribute(attentionTcKernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smemBytes);
  if(e1 != cudaSuccess || e2 != cudaSuccess) { delete p; return nullptr; }
  p->smemBytesPipe = 13 * (size_t)AT_TILE_BYTES + (AT_SK + 512 + AT_REL_MAX + AT_SK) * sizeof(float) + AP_NUM_BARS * 8 + 16 + 1024;
  const int pipeBytes = (int)p->smemBytesPipe;
  e1 = cudaFuncSetAttribute(attentionPipeKernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pipeBytes);
  e2 = cudaFuncSetAttribute(attentionPipeKernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pipeBytes);
  if(e1 == cudaSuccess) e1 = cudaFuncSetAttribute(attentionPipeKernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, pipeBytes);
  if(e2 == cudaSuccess) e2 = cudaFuncSetAttribute(attentionPipeKernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, pipeBytes);
  if(e1 != cudaSuccess || e2 != cudaSuccess) { delete p; return nullptr; }
  int dev = 0;
  p->numSMs = 148;
  if(cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&p->numSMs, cudaDevAttrMultiProcessorCount, dev);
  return p;
}

void attentionTcDestroy(AttnTcPlan* p) { delete p; }

cudaError_t launchAttentionTc(
  cudaStream_t st, const AttnTcPlan* p, int qOff, int kOff, int vOff, int heads, int kvHeads, const float* mask, void* out,
  int outStride, Geom g, int* statusWord, const float2* ropeX, const float2* ropeY, int tableHeads, const float* relBias, int relY, int relX,
  int pipelined) {
  AttnTcArgs a;
  a.g = g; a.heads = heads; a.kvHeads = kvHeads; a.qOff = qOff; a.kOff = kOff; a.vOff = vOff;
  a.keysValid = g.Y * g.RW;
  a.mask = mask; a.out = out; a.outStride = outStride;
  const uint32_t fmt = p->dt == DT_F16 ? 0u : 1u;
  a.idescS = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.idescS256 = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.idescO = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(AT_D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.scaleLog2e = 1.4426950408889634f / sqrtf((float)AT_D);
  a.status = statusWord;
  a.ropeX = ropeX; a.ropeY = ropeY; a.tableHeads = tableHeads;
  a.relBias = relBias; a.relY = relY; a.relX = relX;
  if(relBias && ((2 * relY - 1) * (2 * relX - 1) > AT_REL_MAX || g.X > relX || g.Y > relY)) return cudaErrorInvalidValue;
  // Q and K already rotated (or never rotated): the pipelined kernel, unless the caller asks for the one-CTA-per-
  // (board, head) kernel; the two produce identical bits.
  if(!ropeX && pipelined) {
    const int units = g.n * heads * ((a.keysValid + 127) / 128);
    if(units <= 0) return cudaSuccess;
    dim3 pgrid(units < p->numSMs ? units : p->numSMs);
    if(relBias) {
      if(p->dt == DT_F16) attentionPipeKernel<__half, true><<<pgrid, AP_THREADS, p->smemBytesPipe, st>>>(p->tmQKV, a);
      else attentionPipeKernel<__nv_bfloat16, true><<<pgrid, AP_THREADS, p->smemBytesPipe, st>>>(p->tmQKV, a);
    }
    else {
      if(p->dt == DT_F16) attentionPipeKernel<__half, false><<<pgrid, AP_THREADS, p->smemBytesPipe, st>>>(p->tmQKV, a);
      else attentionPipeKernel<__nv_bfloat16, false><<<pgrid, AP_THREADS, p->smemBytesPipe, st>>>(p->tmQKV, a);
    }
    return cudaGetLastError();
  }
  dim3 grid(g.n * heads);
  if(relBias) {
    if(p->dt == DT_F16) attentionTcKernel<__half, true><<<grid, AT_THREADS, p->smemBytes, st>>>(p->tmQKV, a);
    else attentionTcKernel<__nv_bfloat16, true><<<grid, AT_THREADS, p->smemBytes, st>>>(p->tmQKV, a);
  }
  else {
    if(p->dt == DT_F16) attentionTcKernel<__half, false><<<grid, AT_THREADS, p->smemBytes, st>>>(p->tmQKV, a);
    else attentionTcKernel<__nv_bfloat16, false><<<grid, AT_THREADS, p->smemBytes, st>>>(p->tmQKV, a);
  }
  return cudaGetLastError();
}

}  // namespace kb

#ifdef KB_TC_TRACE
extern "C" int kb_debug_attention_trace(long long* out, int n) { return (int)cudaMemcpyFromSymbol(out, kb::g_atTrace, sizeof(long long) * (n > 256 ? 256 : n)); }
#endif
