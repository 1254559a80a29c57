// Inline-PTX wrappers for the sm_100a features the tensor-core kernels use: mbarriers with bounded waits,
// TMA tile loads/stores, TMEM allocation, tcgen05.mma / commit / ld, and shared-memory matrix descriptors.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

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

// Bounded wait (about 2 s unless another limit is given).  Returns false on time-out or if another role already gave up.
__device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity, volatile int* abortFlag, uint64_t limitNs = 2000000000ull) {
  if(mbarTryWait(bar, parity)) return true;
  const uint64_t t0 = globalTimerNs();
  uint32_t spins = 0;
  while(true) {
    if(mbarTryWait(bar, parity)) return true;
    if((++spins & 63u) == 0u) {
      if(*abortFlag) return false;
      if(globalTimerNs() - t0 > limitNs) return false;
    }
  }
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may start
// while the kernel before it in the stream still runs; it must not touch memory that kernel produces (or still
// reads) before gridDepWait() returns.  gridDepLaunch() lets the next such kernel begin its own preamble.
__device__ __forceinline__ void gridDepWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void gridDepLaunch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void tmaLoad2d(uint32_t dst, const CUtensorMap* tmap, int c0, int c1, uint32_t bar) {
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
    ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
    : "memory");
}

// Tile readiness counters in global memory (per-tile dependencies between consecutive convolutions).
__device__ __forceinline__ uint32_t ldAcquireGpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void redReleaseGpuAdd(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Waits (bounded like mbarWait) until the counters of row tiles lo..hi (at most three) have all reached `target`.
// The polls are relaxed loads that can be in flight together; one acquire fence follows the successful poll.
__device__ __forceinline__ uint32_t ldRelaxedGpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool waitTilesDone(const uint32_t* ctr, int lo, int hi, uint32_t target, volatile int* abortFlag, const volatile int* status) {
  const int mid = lo + 1 <= hi ? lo + 1 : hi;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while(true) {
    const uint32_t v0 = ldRelaxedGpu(ctr + lo), v1 = ldRelaxedGpu(ctr + mid), v2 = ldRelaxedGpu(ctr + hi);
    if(v0 >= target && v1 >= target && v2 >= target) {
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
      return true;
    }
    if(spins == 0) t0 = globalTimerNs();
    if((++spins & 15u) == 0u) {
      // an earlier kernel of the stream that gave up never reports its tiles: do not wait for it
      if(*abortFlag || *status != 0) return false;
      if(globalTimerNs() - t0 > 2000000000ull) return false;
    }
    __nanosleep(64);
  }
}
// All but the n most recent bulk groups of this thread have completed (their global writes included).
__device__ __forceinline__ void bulkWaitPending(int n) {
  switch(n) {
    case 0: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.bulk.wait_group 3;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); break;  // n >= 4: waits for more than asked
  }
}

// shared -> global tile store (asynchronous, tracked by the issuing thread's bulk groups)
__device__ __forceinline__ void tmaStore2d(const CUtensorMap* tmap, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulkWaitRead0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulkWaitRead1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// orders this thread's generic-proxy accesses and its asynchronous-proxy (TMA) accesses in every state space
__device__ __forceinline__ void fenceProxyAsyncAll() { asm volatile("fence.proxy.async;" ::: "memory"); }

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
// Same, with the two shared-memory descriptors given as their low words (start address + leading offset) and the
// high word both share (stride offset, version, swizzle mode); keeps the issuing thread's instruction count low.
__device__ __forceinline__ void ummaLoHi(uint32_t dTmem, uint32_t aLo, uint32_t bLo, uint32_t descHi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
    "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
    "mov.b64 da, {%1, %3};\n\t"
    "mov.b64 db, {%2, %3};\n\t"
    "setp.ne.b32 p, %5, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
    ::"r"(dTmem), "r"(aLo), "r"(bLo), "r"(descHi), "r"(idesc), "r"(accumulate)
    : "memory");
}
// mbarrier arrives once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void ummaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs on neighbouring SMs; cta_group::2).  One MMA instruction, issued by the even CTA,
// computes 256 rows: each CTA supplies its own 128 rows of A and half of the B tile from its own shared memory (at
// the same offsets) and receives its 128 rows of the result in its own TMEM.  Loads of both CTAs signal the even
// CTA's barrier; every load has a single destination.

__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the even CTA of the pair (the cluster window places CTA rank r at
// bit 24 of the shared::cluster address).
__device__ __forceinline__ uint32_t pairLeaderAddr(uint32_t saddr) { return saddr & 0xFEFFFFFFu; }
// Address of the same location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t clusterMapAddr(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// Tile load into this CTA's shared memory whose completion is signalled on a barrier that may live in the pair's
// other CTA (bar is a shared::cluster address).
__device__ __forceinline__ void tmaLoad2dPair(uint32_t dst, const CUtensorMap* tmap, int c0, int c1, uint32_t bar) {
  asm volatile(
    "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
    ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
    : "memory");
}
__device__ __forceinline__ void tmemAllocPair(uint32_t dstSmem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquishPair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDeallocPair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void ummaLoHiPair(uint32_t dTmem, uint32_t aLo, uint32_t bLo, uint32_t descHi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
    "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
    "mov.b64 da, {%1, %3};\n\t"
    "mov.b64 db, {%2, %3};\n\t"
    "setp.ne.b32 p, %5, 0;\n\t"
    "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
    ::"r"(dTmem), "r"(aLo), "r"(bLo), "r"(descHi), "r"(idesc), "r"(accumulate)
    : "memory");
}
// The barrier (a shared::cluster address, in either CTA of the pair) receives one arrival once all MMAs issued so far
// by this thread have completed in both CTAs.
__device__ __forceinline__ void ummaCommitPair(uint32_t clusterBar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(clusterBar) : "memory");
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
// Same wait, naming the 32 destination registers of an earlier load as in/out operands: when the load was issued ahead
// of other work, this ties every later use of the registers to the wait in the compiler's eyes.
__device__ __forceinline__ void tmemLdWaitFor(uint32_t (&r)[32]) {
  asm volatile(
    "tcgen05.wait::ld.sync.aligned;"
    : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
      "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
      "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
      "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
    :
    : "memory");
}

// 32 registers per thread -> 32 lanes x 32 consecutive 32-bit columns (thread t writes lane base+t): the reverse of tmemLd32.
__device__ __forceinline__ void tmemSt32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
    "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
    "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
    "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
    ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
    : "memory");
}
// All earlier tmemSt32 of this thread have been written (needed before the thread reads those columns back).
__device__ __forceinline__ void tmemStWait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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


}  // namespace kb
