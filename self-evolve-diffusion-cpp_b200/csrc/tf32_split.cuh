// Splitting fp32 values into tf32 parts for the tensor cores (kind::tf32 keeps 10 explicit
// mantissa bits and ignores the low 13 bits of the word).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace sdq {

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// x = hi + lo with both parts representable in tf32 (low 13 bits of the word zero).
// Non-finite x: hi carries it, lo is zero.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  hi = round_tf32(x);
  if (fabsf(hi) <= 3.4028234e38f) {
    lo = round_tf32(__fsub_rn(x, hi));
  } else {
    hi = x;
    lo = 0.0f;
  }
}

}  // namespace sdq
