// Row quantization kernels: HBM-bound, one pass over the source.
//
// Activation rows (first half of sd::qgemm, reference src/core/qgemm.cpp:82-96),
// weight rows in the two recipes of the reference (tools/quantize/pack_sdcpp.py:45-51
// and src/core/tensor.cpp:63-78), and the row dequantizer (src/model/ovi_dit.cpp:53-63).
//
// Every fp32 operation that decides an output bit uses an explicit
// round-to-nearest intrinsic (__fdiv_rn, __fmul_rn) so that the compiler can
// neither fuse nor approximate it: the results are bit-identical to the CPU.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <climits>
#include <cstdlib>

#include "sdq_internal.h"

namespace sdq {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide max of non-negative, non-NaN values.  `red` holds kThreads/32 floats.
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protects `red` against the previous row's readers
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < kThreads / 32) ? red[lane] : 0.0f;
  return warp_max(r);
}

// |x| folded into a running max the way std::max(mx, fabs(x)) does: a NaN is skipped.
__device__ __forceinline__ float fold_abs(float mx, float x) { return fmaxf(mx, fabsf(x)); }

// The reference rounds with cvtss2si (src/core/qgemm.cpp:62-69): nearest-even, and
// INT_MIN for NaN or anything outside 32 bits, then clamps to [-127,127].
__device__ __forceinline__ int act_round(float p) {
  int v = (fabsf(p) < 2147483648.0f) ? __float2int_rn(p) : INT_MIN;
  return max(-127, min(127, v));
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
         ((uint32_t)(d & 0xff) << 24);
}

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }

// Programmatic dependent launch: lets the GEMM that follows in the stream (launched with
// the programmatic-serialization attribute) start its prologue -- barrier set-up, tensor
// memory allocation, descriptor prefetch -- while this kernel is still running.  The GEMM
// waits (griddepcontrol.wait) for this whole grid and its writes before it reads anything.
__device__ __forceinline__ void allow_dependent_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- activations: a row lives in registers between the max and the rounding ----
// Requires K % 4 == 0, 16-byte aligned A, K <= kThreads * 4 * VPT.
template <int VPT>
__global__ void __launch_bounds__(kThreads) act_quant_regs(const float* __restrict__ A, int64_t M,
                                                           int64_t K, int8_t* __restrict__ aq,
                                                           float* __restrict__ a_scale) {
  allow_dependent_launch();
  __shared__ float red[kThreads / 32];
  const int k4 = (int)(K >> 2);
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float4* src = reinterpret_cast<const float4*>(A + row * K);
    float4 v[VPT];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < k4) {
        v[i] = ld_stream(src + idx);
        mx = fold_abs(fold_abs(fold_abs(fold_abs(mx, v[i].x), v[i].y), v[i].z), v[i].w);
      }
    }
    mx = block_max(mx, red);
    float sc = __fdiv_rn(mx, 127.0f);
    if (sc == 0.0f) sc = 1.0f;
    if (threadIdx.x == 0) a_scale[row] = sc;
    const float inv = __fdiv_rn(1.0f, sc);
    uint32_t* dst = reinterpret_cast<uint32_t*>(aq + row * K);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < k4)
        dst[idx] = pack4(act_round(__fmul_rn(v[i].x, inv)), act_round(__fmul_rn(v[i].y, inv)),
                         act_round(__fmul_rn(v[i].z, inv)), act_round(__fmul_rn(v[i].w, inv)));
    }
  }
}

// Rows of up to 32*4*VPT elements (K = 3072, the DiT width, with VPT = 24): one WARP per
// row, the row in the warp's registers, no block-wide barrier at all -- shuffles only -- so a
// short row does not pay two __syncthreads per 12 KiB of traffic.
template <int VPT>
__global__ void __launch_bounds__(kThreads) act_quant_warp_rows(const float* __restrict__ A,
                                                                int64_t M, int64_t K,
                                                                int8_t* __restrict__ aq,
                                                                float* __restrict__ a_scale) {
  allow_dependent_launch();
  const int lane = threadIdx.x & 31;
  const int k4 = (int)(K >> 2);
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < M; row += warps) {
    const float4* src = reinterpret_cast<const float4*>(A + row * K);
    float4 v[VPT];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = lane + i * 32;
      if (idx < k4) {
        v[i] = ld_stream(src + idx);
        mx = fold_abs(fold_abs(fold_abs(fold_abs(mx, v[i].x), v[i].y), v[i].z), v[i].w);
      }
    }
    mx = warp_max(mx);
    float sc = __fdiv_rn(mx, 127.0f);
    if (sc == 0.0f) sc = 1.0f;
    if (lane == 0) a_scale[row] = sc;
    const float inv = __fdiv_rn(1.0f, sc);
    uint32_t* dst = reinterpret_cast<uint32_t*>(aq + row * K);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = lane + i * 32;
      if (idx < k4)
        dst[idx] = pack4(act_round(__fmul_rn(v[i].x, inv)), act_round(__fmul_rn(v[i].y, inv)),
                         act_round(__fmul_rn(v[i].z, inv)), act_round(__fmul_rn(v[i].w, inv)));
    }
  }
}

// Any K and alignment: two sweeps over the row (the second is served by L1/L2).
__global__ void __launch_bounds__(kThreads) act_quant_generic(const float* __restrict__ A,
                                                              int64_t M, int64_t K,
                                                              int8_t* __restrict__ aq,
                                                              float* __restrict__ a_scale) {
  allow_dependent_launch();
  __shared__ float red[kThreads / 32];
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float* src = A + row * K;
    float mx = 0.0f;
    for (int64_t k = threadIdx.x; k < K; k += kThreads) mx = fold_abs(mx, src[k]);
    mx = block_max(mx, red);
    float sc = __fdiv_rn(mx, 127.0f);
    if (sc == 0.0f) sc = 1.0f;
    if (threadIdx.x == 0) a_scale[row] = sc;
    const float inv = __fdiv_rn(1.0f, sc);
    int8_t* dst = aq + row * K;
    for (int64_t k = threadIdx.x; k < K; k += kThreads)
      dst[k] = (int8_t)act_round(__fmul_rn(src[k], inv));
  }
}

// ---- LayerNorm + modulation + activation quantization in one pass ----
// The step in front of most DiT linears (reference src/model/blocks.cpp:18-43 without affine
// parameters, then mod_rows, src/model/ovi_dit.cpp:162-173, then the first half of sd::qgemm):
//   ln = (x - mean) * rsqrt(var + eps);  h = ln * (1 + scale[c]) + shift[c];  aq = quantize(h)
// Fusing them deletes the fp32 round trip of `h` (4 bytes/element written and read again).
// The means and variances are block-wide tree sums, not the CPU's left-to-right sums, so
// `h` agrees with the CPU to rounding error (not bit for bit) and an int8 value can differ
// by one step where h lands on a rounding boundary.
// (x - mu) * inv * 1.f + 0.f of blk::layernorm without affine parameters: the multiply by one
// is exact, the add of +0 turns a -0 into +0.
__device__ __forceinline__ float ln_value(float x, float mu, float inv) {
  return __fadd_rn(__fmul_rn(__fsub_rn(x, mu), inv), 0.0f);
}
// Modulated form (mod_rows after a layernorm without parameters): fma(ln, 1 + scale, shift).
// Affine form (blk::layernorm with weight and bias, src/model/blocks.cpp:39-40): the
// reference's build fuses (x - mu) * inv * w + b into fma((x - mu) * inv, w, b).
// `mult` is the column's multiplier from column_multiplier(): 1 + scale, or the weight.
__device__ __forceinline__ float mod_value(float x, float mu, float inv, float mult, float shift,
                                           int affine) {
  if (affine) return fmaf(__fmul_rn(__fsub_rn(x, mu), inv), mult, shift);
  return fmaf(ln_value(x, mu, inv), mult, shift);
}
__device__ __forceinline__ float4 column_multiplier(float4 scale, int affine) {
  if (affine) return scale;
  return make_float4(__fadd_rn(1.0f, scale.x), __fadd_rn(1.0f, scale.y), __fadd_rn(1.0f, scale.z),
                     __fadd_rn(1.0f, scale.w));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < kThreads / 32) ? red[lane] : 0.0f;
  return warp_sum(r);
}

// ---- the reference's own row statistics, bit for bit ----
// blk::layernorm adds the K values of a row left to right in fp32 (mean), then the squared
// deviations left to right (variance): two dependent chains of K additions whose roundings
// no tree sum reproduces.  Here one LANE owns one row and runs the same two chains, so a warp
// carries 32 rows at once; the rows stream through a small ring of shared-memory tiles
// (32 rows x 128 bytes, filled with 16-byte cp.async copies, 16-byte slots XOR-swizzled by
// row so that both the row-major fill and the lane-per-row reads are conflict-free).
// stats[row] = (mean, 1/sqrt(var + eps)).  Two passes over x (HBM-bound); the chains themselves
// cost ~4 cycles per element per row and overlap the copies.
constexpr int kStatStages = 6;
constexpr int kStatWarps = 2;
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__global__ void __launch_bounds__(kStatWarps * 32)
    row_stats_seq_kernel(const float* __restrict__ X, int64_t M, int64_t K, float eps,
                         float2* __restrict__ stats) {
  __shared__ __align__(128) uint8_t ring_mem[kStatWarps * kStatStages * 4096];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = ((int64_t)blockIdx.x * kStatWarps + warp) * 32;
  if (r0 >= M) return;
  const uint32_t ring = smem_addr(ring_mem) + (uint32_t)(warp * kStatStages * 4096);
  const int ntiles = (int)((K + 31) / 32);
  const int sub = lane >> 3, piece = lane & 7;
  const float kf = (float)K;

  auto issue = [&](int t) {  // tile t: columns [32t, 32t+32) of the warp's 32 rows
    if (t < ntiles) {
      const uint32_t st = ring + (uint32_t)((t % kStatStages) * 4096);
      const int64_t col = (int64_t)t * 32 + piece * 4;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int row = i * 4 + sub;
        const bool ok = (r0 + row < M) && (col < K);  // K % 4 == 0: a 16-byte piece is all in or out
        const float* src = ok ? X + (r0 + row) * K + col : X;
        const uint32_t dst = st + (uint32_t)(row * 128 + ((piece ^ (row & 7)) << 4));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0)
                     : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // one group per slot, empty or not
  };

  float mu = 0.0f, acc = 0.0f;
  for (int pass = 0; pass < 2; pass++) {
    acc = 0.0f;
    for (int t = 0; t < kStatStages - 1; t++) issue(t);
    for (int t = 0; t < ntiles; t++) {
      issue(t + kStatStages - 1);  // into the stage every lane finished reading last iteration
      asm volatile("cp.async.wait_group %0;" ::"n"(kStatStages - 1) : "memory");
      __syncwarp();  // every lane's pieces of tile t have landed
      const uint32_t mine = ring + (uint32_t)((t % kStatStages) * 4096 + lane * 128);
      float x[32];
#pragma unroll
      for (int p = 0; p < 8; p++) {
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "r"(mine + (uint32_t)((p ^ (lane & 7)) << 4)));
        x[4 * p] = v.x; x[4 * p + 1] = v.y; x[4 * p + 2] = v.z; x[4 * p + 3] = v.w;
      }
      const int n = (int)min((int64_t)32, K - (int64_t)t * 32);
      if (pass == 0) {
#pragma unroll
        for (int c = 0; c < 32; c++)
          if (c < n) acc = __fadd_rn(acc, x[c]);
      } else {
#pragma unroll
        for (int c = 0; c < 32; c++) {
          if (c < n) {
            const float d = __fsub_rn(x[c], mu);
            acc = __fadd_rn(acc, __fmul_rn(d, d));  // not fused: the reference's build does not fuse it
          }
        }
      }
      __syncwarp();  // the stage may be refilled from the next iteration on
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (pass == 0) mu = __fdiv_rn(acc, kf);
  }
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(acc, kf), eps)));
  if (r0 + lane < M) stats[r0 + lane] = make_float2(mu, inv);
}

template <int VPT>
__global__ void __launch_bounds__(kThreads) ln_mod_quant_regs(const float* __restrict__ X, int64_t M,
                                                              int64_t K, const float* __restrict__ shift,
                                                              const float* __restrict__ scale, float eps,
                                                              int8_t* __restrict__ aq,
                                                              float* __restrict__ a_scale,
                                                              float* __restrict__ h_out,
                                                              const float2* __restrict__ stats,
                                                              int affine) {
  allow_dependent_launch();
  __shared__ float red[kThreads / 32];
  const int k4 = (int)(K >> 2);
  const float inv_n = 1.0f / (float)K;
  // A thread meets the same columns in every row: for short rows their multipliers
  // (1 + scale, or the layernorm's weight) and addends stay in registers across the rows.
  constexpr bool kHoist = VPT <= 3;
  float4 mul_c[kHoist ? VPT : 1], add_c[kHoist ? VPT : 1];
  if (kHoist) {
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < k4) {
        mul_c[i] = column_multiplier(__ldg(reinterpret_cast<const float4*>(scale) + idx), affine);
        add_c[i] = __ldg(reinterpret_cast<const float4*>(shift) + idx);
      }
    }
  }
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float4* src = reinterpret_cast<const float4*>(X + row * K);
    float4 v[VPT];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < k4) {
        v[i] = ld_stream(src + idx);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    float mu, inv;
    if (stats) {  // the reference's left-to-right sums, from row_stats_seq_kernel
      const float2 st = __ldg(stats + row);
      mu = st.x;
      inv = st.y;
    } else {      // block-wide tree sums
      mu = block_sum(s, red) * inv_n;
      float q = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        const int idx = threadIdx.x + i * kThreads;
        if (idx < k4) {
          const float a = v[i].x - mu, b = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
          q += (a * a + b * b) + (c * c + d * d);
        }
      }
      inv = 1.0f / sqrtf(block_sum(q, red) * inv_n + eps);
    }
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < k4) {
        const float4 sc = kHoist ? mul_c[i]
                                 : column_multiplier(__ldg(reinterpret_cast<const float4*>(scale) + idx), affine);
        const float4 sh = kHoist ? add_c[i] : __ldg(reinterpret_cast<const float4*>(shift) + idx);
        v[i].x = mod_value(v[i].x, mu, inv, sc.x, sh.x, affine);
        v[i].y = mod_value(v[i].y, mu, inv, sc.y, sh.y, affine);
        v[i].z = mod_value(v[i].z, mu, inv, sc.z, sh.z, affine);
        v[i].w = mod_value(v[i].w, mu, inv, sc.w, sh.w, affine);
        mx = fold_abs(fold_abs(fold_abs(fold_abs(mx, v[i].x), v[i].y), v[i].z), v[i].w);
        if (h_out) reinterpret_cast<float4*>(h_out + row * K)[idx] = v[i];
      }
    }
    mx = block_max(mx, red);
    float sc = __fdiv_rn(mx, 127.0f);
    if (sc == 0.0f) sc = 1.0f;
    if (threadIdx.x == 0) a_scale[row] = sc;
    const float qinv = __fdiv_rn(1.0f, sc);
    uint32_t* dst = reinterpret_cast<uint32_t*>(aq + row * K);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < k4)
        dst[idx] = pack4(act_round(__fmul_rn(v[i].x, qinv)), act_round(__fmul_rn(v[i].y, qinv)),
                         act_round(__fmul_rn(v[i].z, qinv)), act_round(__fmul_rn(v[i].w, qinv)));
    }
  }
}

// ---- weights ----
template <int DT>
__device__ __forceinline__ float load_src(const void* p, int64_t i);
template <>
__device__ __forceinline__ float load_src<SDQ_F32>(const void* p, int64_t i) {
  return static_cast<const float*>(p)[i];
}
template <>
__device__ __forceinline__ float load_src<SDQ_BF16>(const void* p, int64_t i) {
  // bits << 16, exactly the packer's widening (tools/quantize/pack_sdcpp.py:40-41)
  return __uint_as_float((uint32_t) static_cast<const uint16_t*>(p)[i] << 16);
}
template <>
__device__ __forceinline__ float load_src<SDQ_F16>(const void* p, int64_t i) {
  return __half2float(static_cast<const __half*>(p)[i]);  // exact widening
}

// Round one element under the chosen recipe, given the row's absmax.
template <int MODE>
struct RowRecipe {
  float mul;  // PACKER: 127/safe ; ROWWISE: the divisor sc
  float scale;
  __device__ explicit RowRecipe(float amax) {
    if (MODE == SDQ_MODE_PACKER) {
      const float safe = amax > 0.0f ? amax : 1.0f;
      mul = __fdiv_rn(127.0f, safe);
      scale = __fdiv_rn(amax, 127.0f);
    } else {
      float sc = __fdiv_rn(amax, 127.0f);
      if (sc == 0.0f) sc = 1.0f;
      mul = sc;
      scale = sc;
    }
  }
  __device__ __forceinline__ int q(float x) const {
    if (MODE == SDQ_MODE_PACKER) {
      // np.rint (half to even), then np.clip(-127,127), then astype(int8)
      float r = rintf(__fmul_rn(x, mul));
      r = fminf(fmaxf(r, -127.0f), 127.0f);
      return (int)r;
    } else {
      // std::lround: half away from zero; the int8 cast of the reference does not clamp
      return (int)(int8_t)lroundf(__fdiv_rn(x, mul));
    }
  }
};

// One block per row with the row held in registers between the max and the rounding:
// 16-byte loads (8 bf16/f16 or 4 fp32 elements), packed stores.  Needs last % EPV == 0,
// 16-byte aligned rows, last <= kThreads * EPV * VPT.
template <int DT>
struct Vec {
  static constexpr int EPV = DT == SDQ_F32 ? 4 : 8;  // elements per 16-byte vector
  __device__ static void load(const void* row, int idx, float (&v)[EPV]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(row) + idx);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    if constexpr (DT == SDQ_F32) {
#pragma unroll
      for (int i = 0; i < 4; i++) v[i] = __uint_as_float(w[i]);
    } else if constexpr (DT == SDQ_BF16) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        v[2 * i] = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xffffu)));
        v[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16)));
      }
    }
  }
};

template <int DT, int MODE, int VPT>
__global__ void __launch_bounds__(kThreads) quant_rows_regs(const void* __restrict__ src,
                                                            int64_t rows, int64_t last,
                                                            int8_t* __restrict__ q,
                                                            float* __restrict__ scale) {
  constexpr int EPV = Vec<DT>::EPV;
  constexpr int ESZ = DT == SDQ_F32 ? 4 : 2;
  __shared__ float red[kThreads / 32];
  const int nvec = (int)(last / EPV);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const char* rp = static_cast<const char*>(src) + row * last * ESZ;
    float v[VPT][EPV];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < nvec) {
        Vec<DT>::load(rp, idx, v[i]);
#pragma unroll
        for (int e = 0; e < EPV; e++) mx = fmaxf(mx, fabsf(v[i][e]));
      }
    }
    mx = block_max(mx, red);
    const RowRecipe<MODE> rr(mx);
    if (threadIdx.x == 0) scale[row] = rr.scale;
    int8_t* qp = q + row * last;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < nvec) {
        uint32_t w0 = pack4(rr.q(v[i][0]), rr.q(v[i][1]), rr.q(v[i][2]), rr.q(v[i][3]));
        if constexpr (EPV == 4) {
          reinterpret_cast<uint32_t*>(qp)[idx] = w0;
        } else {
          uint32_t w1 = pack4(rr.q(v[i][EPV - 4]), rr.q(v[i][EPV - 3]), rr.q(v[i][EPV - 2]), rr.q(v[i][EPV - 1]));
          reinterpret_cast<uint2*>(qp)[idx] = make_uint2(w0, w1);
        }
      }
    }
  }
}

// One block per row (grid-stride), two sweeps.  `last` any size.
template <int DT, int MODE>
__global__ void __launch_bounds__(kThreads) quant_rows_block(const void* __restrict__ src,
                                                             int64_t rows, int64_t last,
                                                             int8_t* __restrict__ q,
                                                             float* __restrict__ scale) {
  __shared__ float red[kThreads / 32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t base = row * last;
    float mx = 0.0f;
    for (int64_t k = threadIdx.x; k < last; k += kThreads) {
      const float f = fabsf(load_src<DT>(src, base + k));
      // PACKER: np.abs(x).max() ; ROWWISE: std::max(mx, std::abs(w)) -- equal for finite rows
      mx = fmaxf(mx, f);
    }
    mx = block_max(mx, red);
    const RowRecipe<MODE> rr(mx);
    if (threadIdx.x == 0) scale[row] = rr.scale;
    for (int64_t k = threadIdx.x; k < last; k += kThreads)
      q[base + k] = (int8_t)rr.q(load_src<DT>(src, base + k));
  }
}

// One warp per row for short rows (last <= 64), e.g. conv kernels with rows of 7 or 2.
template <int DT, int MODE>
__global__ void __launch_bounds__(kThreads) quant_rows_warp(const void* __restrict__ src,
                                                            int64_t rows, int64_t last,
                                                            int8_t* __restrict__ q,
                                                            float* __restrict__ scale) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_per_grid = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < rows;
       row += warps_per_grid) {
    const int64_t base = row * last;
    float mx = 0.0f;
    for (int64_t k = lane; k < last; k += 32) mx = fmaxf(mx, fabsf(load_src<DT>(src, base + k)));
    mx = warp_max(mx);
    const RowRecipe<MODE> rr(mx);
    if (lane == 0) scale[row] = rr.scale;
    for (int64_t k = lane; k < last; k += 32)
      q[base + k] = (int8_t)rr.q(load_src<DT>(src, base + k));
  }
}

__global__ void __launch_bounds__(kThreads) dequant_rows_kernel(const int8_t* __restrict__ q,
                                                                const float* __restrict__ scale,
                                                                int64_t numel, int64_t last,
                                                                float* __restrict__ w) {
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < numel;
       i += (int64_t)gridDim.x * kThreads)
    w[i] = __fmul_rn((float)q[i], scale[i / last]);
}

template <int DT, int MODE>
cudaError_t launch_quant_t(const void* src, int64_t rows, int64_t last, int8_t* q, float* scale,
                           int sm_count, cudaStream_t s) {
  if (last <= 64) {
    int64_t blocks = (rows + kThreads / 32 - 1) / (kThreads / 32);
    if (blocks > (int64_t)sm_count * 32) blocks = (int64_t)sm_count * 32;
    quant_rows_warp<DT, MODE><<<(unsigned)blocks, kThreads, 0, s>>>(src, rows, last, q, scale);
  } else {
    int64_t blocks = rows < (int64_t)sm_count * 8 ? rows : (int64_t)sm_count * 8;
    constexpr int EPV = Vec<DT>::EPV;
    const bool vec = (last % EPV == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
    const int64_t per_thread = (last / EPV + kThreads - 1) / kThreads;
    if (vec && per_thread <= 2)
      quant_rows_regs<DT, MODE, 2><<<(unsigned)blocks, kThreads, 0, s>>>(src, rows, last, q, scale);
    else if (vec && per_thread <= 4)
      quant_rows_regs<DT, MODE, 4><<<(unsigned)blocks, kThreads, 0, s>>>(src, rows, last, q, scale);
    else if (vec && per_thread <= 8)
      quant_rows_regs<DT, MODE, 8><<<(unsigned)blocks, kThreads, 0, s>>>(src, rows, last, q, scale);
    else
      quant_rows_block<DT, MODE><<<(unsigned)blocks, kThreads, 0, s>>>(src, rows, last, q, scale);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_act_quant(const float* A, int64_t M, int64_t K, int8_t* aq, float* a_scale,
                             int sm_count, cudaStream_t s) {
  if (M <= 0 || K <= 0) return cudaSuccess;
  // 8 resident blocks of 256 threads fill an SM; rows beyond that are strided over.
  int64_t blocks = M < (int64_t)sm_count * 8 ? M : (int64_t)sm_count * 8;
  const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(aq) & 3) == 0);
  const int64_t per_thread = (K / 4 + kThreads - 1) / kThreads;  // float4 per thread
  count_launch();
  // One warp per row pays off once there are many rows per SM (measured at K = 3072: 98 vs 109 us
  // at 27280 rows, equal at 13824, 17.5 vs 15.1 us at 3584 rows, where one block per row spreads
  // the few rows better); SDQ_ACTQ_WARP_MIN_ROWS overrides the threshold for measurements.
  const char* wmin_env = getenv("SDQ_ACTQ_WARP_MIN_ROWS");
  const int64_t warp_min_rows = wmin_env ? atoll(wmin_env) : (int64_t)sm_count * 80;
  if (vec && K <= 32 * 4 * 24 && M >= warp_min_rows) {
    int64_t wblocks = (M + kThreads / 32 - 1) / (kThreads / 32);
    if (wblocks > (int64_t)sm_count * 4) wblocks = (int64_t)sm_count * 4;
    if (K <= 32 * 4 * 8)
      act_quant_warp_rows<8><<<(unsigned)wblocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
    else
      act_quant_warp_rows<24><<<(unsigned)wblocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
  } else if (vec && per_thread <= 3) {
    act_quant_regs<3><<<(unsigned)blocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
  } else if (vec && per_thread <= 6) {
    act_quant_regs<6><<<(unsigned)blocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
  } else if (vec && per_thread <= 14) {
    act_quant_regs<14><<<(unsigned)blocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
  } else if (vec && per_thread <= 18) {
    act_quant_regs<18><<<(unsigned)blocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
  } else {
    act_quant_generic<<<(unsigned)blocks, kThreads, 0, s>>>(A, M, K, aq, a_scale);
  }
  return cudaGetLastError();
}

cudaError_t launch_ln_mod_quant(const float* X, int64_t M, int64_t K, const float* shift,
                                const float* scale, float eps, int8_t* aq, float* a_scale,
                                float* h_out, float2* stats, int affine, int sm_count,
                                cudaStream_t s) {
  if (M <= 0 || K <= 0) return cudaSuccess;
  const int64_t per_thread = (K / 4 + kThreads - 1) / kThreads;
  const bool ok = (K % 4 == 0) && per_thread <= 16 && ((reinterpret_cast<uintptr_t>(X) & 15) == 0) &&
                  ((reinterpret_cast<uintptr_t>(shift) & 15) == 0) &&
                  ((reinterpret_cast<uintptr_t>(scale) & 15) == 0) &&
                  ((reinterpret_cast<uintptr_t>(aq) & 3) == 0) &&
                  (!h_out || (reinterpret_cast<uintptr_t>(h_out) & 15) == 0);
  if (!ok) return cudaErrorInvalidValue;
  if (stats) {
    if ((reinterpret_cast<uintptr_t>(stats) & 7) != 0) return cudaErrorInvalidValue;
    const int64_t groups = (M + 31) / 32;
    count_launch();
    row_stats_seq_kernel<<<(unsigned)((groups + kStatWarps - 1) / kStatWarps), kStatWarps * 32, 0, s>>>(
        X, M, K, eps, stats);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  count_launch();
  int64_t blocks = M < (int64_t)sm_count * 8 ? M : (int64_t)sm_count * 8;
  if (per_thread <= 3)
    ln_mod_quant_regs<3><<<(unsigned)blocks, kThreads, 0, s>>>(X, M, K, shift, scale, eps, aq, a_scale, h_out, stats, affine);
  else if (per_thread <= 8)
    ln_mod_quant_regs<8><<<(unsigned)blocks, kThreads, 0, s>>>(X, M, K, shift, scale, eps, aq, a_scale, h_out, stats, affine);
  else
    ln_mod_quant_regs<16><<<(unsigned)blocks, kThreads, 0, s>>>(X, M, K, shift, scale, eps, aq, a_scale, h_out, stats, affine);
  return cudaGetLastError();
}

cudaError_t launch_quantize_rows(const void* src, int src_dtype, int64_t rows, int64_t last,
                                 int mode, int8_t* q, float* scale, int sm_count,
                                 cudaStream_t s) {
  if (rows <= 0 || last <= 0) return cudaSuccess;
  count_launch();
  if (mode == SDQ_MODE_ROWWISE) {
    if (src_dtype != SDQ_F32) return cudaErrorInvalidValue;
    return launch_quant_t<SDQ_F32, SDQ_MODE_ROWWISE>(src, rows, last, q, scale, sm_count, s);
  }
  switch (src_dtype) {
    case SDQ_F32: return launch_quant_t<SDQ_F32, SDQ_MODE_PACKER>(src, rows, last, q, scale, sm_count, s);
    case SDQ_BF16: return launch_quant_t<SDQ_BF16, SDQ_MODE_PACKER>(src, rows, last, q, scale, sm_count, s);
    case SDQ_F16: return launch_quant_t<SDQ_F16, SDQ_MODE_PACKER>(src, rows, last, q, scale, sm_count, s);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_dequant_rows(const int8_t* q, const float* scale, int64_t rows, int64_t last,
                                float* w, int sm_count, cudaStream_t s) {
  const int64_t numel = rows * last;
  if (numel <= 0) return cudaSuccess;
  int64_t blocks = (numel + kThreads - 1) / kThreads;
  if (blocks > (int64_t)sm_count * 16) blocks = (int64_t)sm_count * 16;
  count_launch();
  dequant_rows_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(q, scale, numel, last, w);
  return cudaGetLastError();
}

}  // namespace sdq
