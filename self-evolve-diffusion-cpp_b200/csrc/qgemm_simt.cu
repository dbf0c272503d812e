// Portable CUDA-core int8 GEMM + rescale epilogue for shapes the tensor-core
// kernel does not take (K not a multiple of 16, unaligned operands), e.g. the
// reference's own odd test shape (17,31,13) (tests/test_core.cpp:95).  It keeps
// sd::qgemm total on the device; it is not the fast path.
#include "sdq_internal.h"
#include "epilogue.cuh"

namespace sdq {
namespace {

constexpr int TM = 32, TN = 32, TK = 64;

// 256 threads, each owns a 2x2 patch of the 32x32 output tile.
__global__ void __launch_bounds__(256) qgemm_simt_kernel(GemmArgs g) {
  __shared__ int8_t sa[TM][TK + 4];
  __shared__ int8_t sb[TN][TK + 4];
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  int32_t acc[2][2] = {{0, 0}, {0, 0}};
  for (int64_t k0 = 0; k0 < g.K; k0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      const int r = e / TK, c = e % TK;
      const int64_t gm = m0 + r, gn = n0 + r, gk = k0 + c;
      sa[r][c] = (gm < g.M && gk < g.K) ? g.aq[gm * g.K + gk] : (int8_t)0;
      sb[r][c] = (gn < g.N && gk < g.K) ? g.bq[gn * g.K + gk] : (int8_t)0;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < TK; k++) {
      const int a0 = sa[ty * 2][k], a1 = sa[ty * 2 + 1][k];
      const int b0 = sb[tx * 2][k], b1 = sb[tx * 2 + 1][k];
      acc[0][0] += a0 * b0;
      acc[0][1] += a0 * b1;
      acc[1][0] += a1 * b0;
      acc[1][1] += a1 * b1;
    }
    __syncthreads();
  }
  const bool gelu = (g.flags & SDQ_GELU_TANH) != 0;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int64_t gm = m0 + ty * 2 + i;
    if (gm >= g.M) continue;
    const float as = g.a_scale[gm];
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int64_t gn = n0 + tx * 2 + j;
      if (gn >= g.N) continue;
      if (g.acc_dump) g.acc_dump[gm * g.N + gn] = acc[i][j];
      float o = epilogue_value(acc[i][j], as, g.b_scale[gn], g.bias ? g.bias + gn : nullptr, gelu);
      if (g.residual) o = residual_value(o, g.residual[gm * g.N + gn], g.gate ? g.gate + gn : nullptr);
      g.out[gm * g.N + gn] = o;
    }
  }
}

}  // namespace

cudaError_t launch_qgemm_simt(const GemmArgs& g, cudaStream_t s) {
  if (g.M <= 0 || g.N <= 0) return cudaSuccess;
  dim3 grid((unsigned)((g.N + TN - 1) / TN), (unsigned)((g.M + TM - 1) / TM));
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  count_launch();
  qgemm_simt_kernel<<<grid, 256, 0, s>>>(g);
  return cudaGetLastError();
}

}  // namespace sdq
