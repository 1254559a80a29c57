// Device-side pieces shared by the tensor-core convolution kernels (kb_conv_tc.cu, kb_conv_fused.cu): activations
// evaluated stage by stage on packed fp32 pairs, packing to and from the storage type, TMEM loads.
#pragma once

#include "kb_kernels.cuh"
#include "kb_tc_ptx.cuh"
#include "kb_act.cuh"
#include "../../include/kb_modelblob.h"

namespace kb {

// ---------------------------------------------------------------------------------------------
// Fast activations for the reduced-precision epilogue

// G values at once, stage by stage, so that G independent dependency chains are in flight per thread: the special
// function unit has a long latency and an epilogue warp has only one other warp to share its scheduler with.
template <int ACT, int G>
__device__ __forceinline__ void actStaged(float (&x)[G]) {
  if(ACT == KB_ACT_RELU) {
#pragma unroll
    for(int i = 0; i < G; i++) x[i] = fmaxf(x[i], 0.0f);
  }
  else if(ACT == KB_ACT_MISH || ACT == KB_ACT_MISH_SCALE8) {
    const float kk = (ACT == KB_ACT_MISH ? 1.0f : 8.0f) * 1.4426950408889634f;
    float n[G];
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = x[i] * kk;
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = ex2Approx(n[i]);
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = fmaf(n[i], n[i] + 2.0f, 2.0f);
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = rcpApprox(n[i]);
#pragma unroll
    for(int i = 0; i < G; i++) x[i] = fmaf(-2.0f, x[i] * n[i], x[i]);
  }
  else if(ACT == KB_ACT_SILU) {
    float n[G];
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = x[i] * -1.4426950408889634f;
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = ex2Approx(n[i]);
#pragma unroll
    for(int i = 0; i < G; i++) n[i] = rcpApprox(1.0f + n[i]);
#pragma unroll
    for(int i = 0; i < G; i++) x[i] *= n[i];
  }
}

// The same on pairs of values with the packed fp32 instructions of sm_100 (two IEEE operations per instruction, half
// the issue slots; results are bit-identical to the scalar form).  The special-function calls stay scalar.
template <int ACT, int G2>
__device__ __forceinline__ void actStaged2(float2 (&x)[G2]) {
  if(ACT == KB_ACT_RELU) {
#pragma unroll
    for(int i = 0; i < G2; i++) { x[i].x = fmaxf(x[i].x, 0.0f); x[i].y = fmaxf(x[i].y, 0.0f); }
  }
  else if(ACT == KB_ACT_MISH || ACT == KB_ACT_MISH_SCALE8) {
    const float kk = (ACT == KB_ACT_MISH ? 1.0f : 8.0f) * 1.4426950408889634f;
    // x - 2x / (n^2 + 2n + 2) = x - x / q with q = n^2/2 + n + 1 = n * (n/2 + 1) + 1.  The code computes -q (negated
    // constants), so that the reciprocal comes out negated and the last step is one fused multiply-add without a
    // separate negation: x + x * (-1/q).
    const float2 kk2 = make_float2(kk, kk), half2v = make_float2(-0.5f, -0.5f), one = make_float2(-1.0f, -1.0f);
    float2 n[G2];
#pragma unroll
    for(int i = 0; i < G2; i++) n[i] = __fmul2_rn(x[i], kk2);
#pragma unroll
    for(int i = 0; i < G2; i++) { n[i].x = ex2Approx(n[i].x); n[i].y = ex2Approx(n[i].y); }
#pragma unroll
    for(int i = 0; i < G2; i++) n[i] = __ffma2_rn(n[i], __ffma2_rn(n[i], half2v, one), one);
#pragma unroll
    for(int i = 0; i < G2; i++) { n[i].x = rcpApprox(n[i].x); n[i].y = rcpApprox(n[i].y); }
#pragma unroll
    for(int i = 0; i < G2; i++) x[i] = __ffma2_rn(x[i], n[i], x[i]);
  }
  else if(ACT == KB_ACT_SILU) {
    const float2 kk2 = make_float2(-1.4426950408889634f, -1.4426950408889634f), one = make_float2(1.0f, 1.0f);
    float2 n[G2];
#pragma unroll
    for(int i = 0; i < G2; i++) n[i] = __fmul2_rn(x[i], kk2);
#pragma unroll
    for(int i = 0; i < G2; i++) { n[i].x = ex2Approx(n[i].x); n[i].y = ex2Approx(n[i].y); }
#pragma unroll
    for(int i = 0; i < G2; i++) n[i] = __fadd2_rn(one, n[i]);
#pragma unroll
    for(int i = 0; i < G2; i++) { n[i].x = rcpApprox(n[i].x); n[i].y = rcpApprox(n[i].y); }
#pragma unroll
    for(int i = 0; i < G2; i++) x[i] = __fmul2_rn(x[i], n[i]);
  }
}

template <typename T> struct Pack2;
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
  // v + (the two packed values of u), with the mixed-precision add of sm_100 (exact conversion, one rounding)
  static __device__ __forceinline__ float2 addTo(uint32_t u, float2 v) {
    float2 o;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; add.rn.f32.f16 %0, lo, %3; add.rn.f32.f16 %1, hi, %4; }"
        : "=f"(o.x), "=f"(o.y) : "r"(u), "f"(v.x), "f"(v.y));
    return o;
  }
};
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
  static __device__ __forceinline__ float2 addTo(uint32_t u, float2 v) {
    float2 o;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; add.rn.f32.bf16 %0, lo, %3; add.rn.f32.bf16 %1, hi, %4; }"
        : "=f"(o.x), "=f"(o.y) : "r"(u), "f"(v.x), "f"(v.y));
    return o;
  }
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

}  // namespace kb
