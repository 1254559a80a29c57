// Fast activation functions for reduced-precision outputs (fp16 / bf16): special-function-unit approximations whose
// error is far below the output rounding.  The fp32 paths use the accurate library functions instead.
#pragma once

#include "../../include/kb_modelblob.h"

namespace kb {

__device__ __forceinline__ float ex2Approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcpApprox(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// mish(x) = x*tanh(softplus(x)) = x - 2x / (n^2 + 2n + 2) with n = e^x (exact identity).  Large x: n = inf, the
// reciprocal is 0 and the result is x; very negative x: n = 0 and the result is 0.  No clamp is needed.
__device__ __forceinline__ float fastMish(float x) {
  const float n = ex2Approx(x * 1.4426950408889634f);
  const float r = rcpApprox(fmaf(n, n + 2.0f, 2.0f));
  return fmaf(-2.0f, x * r, x);
}
__device__ __forceinline__ float fastAct(float x, int act) {
  switch(act) {
    case KB_ACT_RELU: return fmaxf(x, 0.0f);
    case KB_ACT_MISH: return fastMish(x);
    case KB_ACT_SILU: return x * rcpApprox(1.0f + ex2Approx(x * -1.4426950408889634f));
    case KB_ACT_MISH_SCALE8: {
      const float n = ex2Approx(x * (8.0f * 1.4426950408889634f));
      const float r = rcpApprox(fmaf(n, n + 2.0f, 2.0f));
      return fmaf(-2.0f, x * r, x);
    }
    default: return x;
  }
}

}  // namespace kb
