// The fp32 epilogue shared by the GEMM kernels.
#pragma once
#include <cuda_runtime.h>

namespace sdq {

// GELU, tanh form (reference src/model/ovi_dit.cpp:132-142):
//   0.5 v (1 + tanh(u)),  u = 0.79788456 (v + 0.044715 v^3).
// Since 0.5 (1 + tanh(u)) = 1 / (1 + exp(-2u)), it is evaluated as v * rcp(1 + ex2(-2u log2 e))
// with the hardware ex2/rcp approximations: ~1e-6 absolute from libm's tanhf, far inside
// the 1e-3 bound this fused activation is held to (the CPU's own std::tanh is not
// bit-reproducible across libms either).
__device__ __forceinline__ float gelu_tanh(float v) {
  const float p = fmaf(0.044715f * v * v, v, v);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(p * (-2.0f * 0.7978845608028654f * 1.4426950408889634f)));
  return __fdividef(v, 1.0f + e);
}

// out = (float)acc * (a_scale * b_scale)   (reference src/core/qgemm.cpp:123-124,135):
// int -> float conversion rounds to nearest even, the scales are multiplied
// first, then one more multiply; explicit _rn intrinsics keep the compiler from
// re-associating or fusing, so this value is bit-identical to the CPU's.
__device__ __forceinline__ float rescale(int acc, float a_scale, float b_scale) {
  return __fmul_rn(__int2float_rn(acc), __fmul_rn(a_scale, b_scale));
}

__device__ __forceinline__ float epilogue_value(int acc, float a_scale, float b_scale,
                                                const float* bias, bool gelu) {
  float o = rescale(acc, a_scale, b_scale);
  if (bias) o = __fadd_rn(o, *bias);  // y[i,j] += b[j], reference src/model/ovi_dit.cpp:71-79
  if (gelu) o = gelu_tanh(o);
  return o;
}

// The residual update the reference's callers run on a linear's output y:
//   x[i,j] += y[i,j] * gate[j]   (gated_add_inplace, reference src/model/ovi_dit.cpp:152-159)
//   x[i,j] += y[i,j]             (add_inplace, reference src/model/ovi_dit.cpp:144-149)
// The reference is built -O3 for an FMA target and GCC contracts the first form into one fused
// multiply-add (checked against the compiled function), so fmaf is the bit-exact form here.
__device__ __forceinline__ float residual_value(float y, float x, const float* gate) {
  return gate ? fmaf(y, *gate, x) : __fadd_rn(x, y);
}

}  // namespace sdq
