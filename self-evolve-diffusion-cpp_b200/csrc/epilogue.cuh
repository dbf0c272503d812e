// The fp32 epilogue shared by the GEMM kernels.
#pragma once
#include <cuda_runtime.h>

namespace sdq {

// GELU, tanh form (reference src/model/ovi_dit.cpp:132-142).  tanh(u) is
// evaluated as 1 - 2/(1+exp(2u)); it agrees with libm's tanhf to ~1e-6
// absolute, far inside the 1e-3 bound this fused activation is held to (the
// CPU's own std::tanh is not bit-reproducible across libms either).
__device__ __forceinline__ float gelu_tanh(float v) {
  const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
  return 0.5f * v * (1.0f + t);
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

}  // namespace sdq
