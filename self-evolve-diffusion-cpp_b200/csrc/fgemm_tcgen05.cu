// fp32 matmul on the Blackwell tensor cores: C[M,N] = A[M,K] * W[K,N] (+ bias[N]), the
// reference's sd::matmul (src/core/gemm.cpp:115-160) behind blk::linear (src/model/blocks.cpp:15)
// for the linears that are NOT int8 in a pack (small or preserved tensors) and for unpacked
// fp32 checkpoints.
//
// The tensor cores have no fp32 input type; kind::tf32 keeps 10 mantissa bits.  Each operand is
// therefore split into two tf32 numbers, x = hi + lo with hi = tf32(x) and lo = tf32(x - hi),
// and every product is issued as three MMAs into one fp32 accumulator,
//     hi*hi + hi*lo + lo*hi          (the dropped lo*lo term is ~2^-22 of the product),
// which removes the input rounding at a third of the tf32 rate.  The tensor core's accumulator
// truncates, so a long chain of accumulations drifts (measured 7e-9 * K of the largest output
// when all of K goes into one accumulator); the sum is therefore cut into groups of kFGroup
// k-blocks (256 elements): each group is accumulated in tensor memory, then added into fp32
// registers by the epilogue warps with IEEE additions while the next group's MMAs run into the
// other accumulator buffer.  The reference's own result depends on its BLAS / SIMD summation
// order, so this path is held to the reference's tolerance for matmul (max-abs error / max-abs
// output <= 1e-3, tests/test_core.cpp:82-84), not to bit equality.
//
// Layout: A_hi / A_lo are [M,K] fp32 planes written by split_tf32_kernel; the weight is
// transposed once at upload into [N,K] planes W_hi / W_lo (K-major "TN" operands, as in the
// int8 kernels).  One persistent CTA per SM, 320 threads, the same roles and the same bounded
// mbarrier waits as qgemm_tc_kernel: a TMA producer lane (four 128-byte-swizzled tiles per
// 32-element k-block), an MMA lane (4 k-steps x 3 products per stage), eight epilogue warps
// (tcgen05.ld, + bias, staged bulk tensor stores), two accumulator buffers in tensor memory.
#include "tc_common.cuh"
#include "tf32_split.cuh"

namespace sdq {
namespace {
using namespace tc;

constexpr int kFBlockN = 128;
constexpr int kFBlockK = 32;   // fp32 elements: one 128-byte swizzle row
constexpr int kFStages = 3;
constexpr int kFGroup = 8;     // k-blocks per accumulation group (256 elements of K)
constexpr int kFTile = BLOCK_M * kFBlockK * 4;  // 16 KiB; the four operand tiles have this size
constexpr int kFStageBytes = 4 * kFTile;
constexpr int kFTmemCols = 2 * kFBlockN;
constexpr int kFSmemBytes = kFStages * kFStageBytes + 8 * 4096 + 256 + 1024;
// instruction descriptor: D = f32 (1 << 4), A = B = tf32 (2 << 7, 2 << 10), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t kFIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kFBlockN >> 3) << 17) |
                             ((uint32_t)(BLOCK_M >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct FGemmArgs {
  int64_t M, N, K;
  const float* bias;  // [N] or null
  float* out;         // [M,N]
  int* status;
};

__global__ void __launch_bounds__(kNumThreads, 1)
    fgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a_hi,
                    const __grid_constant__ CUtensorMap tmap_a_lo,
                    const __grid_constant__ CUtensorMap tmap_b_hi,
                    const __grid_constant__ CUtensorMap tmap_b_lo,
                    const __grid_constant__ CUtensorMap tmap_out, int use_tma_store, FGemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_staging = base + kFStages * kFStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kFStages * kFStageBytes + 8 * 4096);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kFStages;
  const uint32_t bar_tfull = bar_empty + 8 * kFStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kFStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m_blocks = (int)((g.M + BLOCK_M - 1) / BLOCK_M);
  const int num_n_blocks = (int)((g.N + kFBlockN - 1) / kFBlockN);
  const int num_k_blocks = (int)((g.K + kFBlockK - 1) / kFBlockK);
  const int num_tiles = num_m_blocks * num_n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kFStages; s++) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 8);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tmap_a_hi);
    prefetch_tmap(&tmap_a_lo);
    prefetch_tmap(&tmap_b_hi);
    prefetch_tmap(&tmap_b_lo);
    if (use_tma_store) prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kFTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer
      grid_dependency_wait();  // the A planes come from the split kernel launched just before
      const uint64_t keep_policy = policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, num_m_blocks, num_n_blocks, m_blk, n_blk);
        for (int kb = 0; kb < num_k_blocks; kb++) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x500 | 1);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t st = base + stage * kFStageBytes;
          mbar_expect_tx(full, kFStageBytes);
          tma_load_2d(st, &tmap_a_hi, full, kb * kFBlockK, m_blk * BLOCK_M);
          tma_load_2d(st + kFTile, &tmap_a_lo, full, kb * kFBlockK, m_blk * BLOCK_M);
          tma_load_2d_hint(st + 2 * kFTile, &tmap_b_hi, full, kb * kFBlockK, n_blk * kFBlockN, keep_policy);
          tma_load_2d_hint(st + 3 * kFTile, &tmap_b_lo, full, kb * kFBlockK, n_blk * kFBlockN, keep_policy);
          if (++stage == kFStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuer
      uint32_t stage = 0, phase = 0, abuf = 0, aphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb0 = 0; ok && kb0 < num_k_blocks; kb0 += kFGroup) {
          // one accumulation group into one of the two accumulator buffers
          ok = mbar_wait(bar_tempty + 8 * abuf, aphase ^ 1u, abort_flag, g.status, 0x600 | 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + abuf * kFBlockN;
          const int kb1 = min(kb0 + kFGroup, num_k_blocks);
          for (int kb = kb0; kb < kb1; kb++) {
            ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 0x600 | 2);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = base + stage * kFStageBytes;
            const uint64_t a_hi = make_smem_desc(st), a_lo = make_smem_desc(st + kFTile);
            const uint64_t b_hi = make_smem_desc(st + 2 * kFTile), b_lo = make_smem_desc(st + 3 * kFTile);
#pragma unroll
            for (int k = 0; k < kFBlockK / 8; k++) {
              // one kind::tf32 instruction covers 8 elements = 32 bytes of K: +2 in the address field
              const uint64_t o = (uint64_t)(k * 2);
              umma_tf32(tmem_d, a_lo + o, b_hi + o, kFIdesc, (uint32_t)(((kb - kb0) | k) != 0));  // small terms first
              umma_tf32(tmem_d, a_hi + o, b_lo + o, kFIdesc, 1u);
              umma_tf32(tmem_d, a_hi + o, b_hi + o, kFIdesc, 1u);
            }
            umma_commit(bar_empty + 8 * stage);
            if (++stage == kFStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          umma_commit(bar_tfull + 8 * abuf);
          abuf ^= 1u;
          if (abuf == 0) aphase ^= 1u;
        }
      }
    }
  } else {
    // -------------------------------------------------- epilogue (8 warps)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t box = smem_staging + (uint32_t)((warp - 2) * 4096);
    const uint64_t stream_policy = policy_evict_first();
    uint32_t abuf = 0, aphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, num_m_blocks, num_n_blocks, m_blk, n_blk);
      const int64_t row0 = (int64_t)m_blk * BLOCK_M + quarter * 32;
      const int64_t row = row0 + lane;
      const int64_t n0 = (int64_t)n_blk * kFBlockN;
      // this warp's two 32-column chunks of the tile, summed over the groups in registers
      float acc[2][32];
#pragma unroll
      for (int c = 0; c < 2; c++)
#pragma unroll
        for (int j = 0; j < 32; j++) acc[c][j] = 0.0f;
      for (int kb0 = 0; ok && kb0 < num_k_blocks; kb0 += kFGroup) {
        ok = mbar_wait_warp(bar_tfull + 8 * abuf, aphase, abort_flag, g.status, 0x700 | 1);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + abuf * kFBlockN + (half + 2 * c) * 32 + ((uint32_t)(quarter * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) acc[c][j] = __fadd_rn(acc[c][j], __uint_as_float(r[j]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * abuf);
        abuf ^= 1u;
        if (abuf == 0) aphase ^= 1u;
      }
      if (!ok) break;
      if (row0 < g.M) {
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int64_t nc = n0 + (half + 2 * c) * 32;
          if (nc >= g.N) break;
          float (&o)[32] = acc[c];
          if (g.bias) {  // C += bias as a separate add, like add_bias (src/core/gemm.cpp:33-40)
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (nc + j < g.N) o[j] = __fadd_rn(o[j], __ldg(g.bias + nc + j));
          }
          if (use_tma_store) {
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              st_shared_v4(box + (uint32_t)(lane * 128 + (((j >> 2) ^ (lane & 7)) << 4)),
                           make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]));
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d_hint(&tmap_out, box, (int)nc, (int)row0, stream_policy);
              bulk_commit();
            }
          } else if (row < g.M) {
            float* out_row = g.out + row * g.N;
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (nc + j < g.N) out_row[nc + j] = o[j];
          }
        }
      }
    }
  }

  // ---------------------------------------------------- common exit
  if (warp >= 2 && lane == 0) bulk_wait_read<0>();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);  // let bulk copies in flight land (~1 ms)
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, kFTmemCols);
  }
}

__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ x, int64_t n,
                                                         float* __restrict__ hi,
                                                         float* __restrict__ lo) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256)
    split_tf32(x[i], hi[i], lo[i]);
}

// W [K,N] row-major (the reference's blk::Linear layout, src/model/blocks.h:22-30) ->
// transposed planes hi / lo [N,K]: 32x32 tiles through shared memory, both sides coalesced.
__global__ void __launch_bounds__(256) transpose_split_kernel(const float* __restrict__ w, int64_t K,
                                                              int64_t N, float* __restrict__ hi,
                                                              float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t k0 = (int64_t)blockIdx.y * 32, n0 = (int64_t)blockIdx.x * 32;
  for (int r = ty; r < 32; r += 8)
    tile[r][tx] = (k0 + r < K && n0 + tx < N) ? w[(k0 + r) * N + n0 + tx] : 0.0f;
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    if (n0 + r < N && k0 + tx < K) {
      float h, l;
      split_tf32(tile[tx][r], h, l);
      hi[(n0 + r) * K + k0 + tx] = h;
      lo[(n0 + r) * K + k0 + tx] = l;
    }
  }
}

// Any shape (K % 4 != 0, unaligned pointers): one thread per output, fp32 FMA chain over k.
__global__ void __launch_bounds__(256) fgemm_simt_kernel(const float* __restrict__ a,
                                                         const float* __restrict__ w_hi,
                                                         const float* __restrict__ w_lo, int64_t M,
                                                         int64_t N, int64_t K,
                                                         const float* __restrict__ bias,
                                                         float* __restrict__ out) {
  const int64_t total = M * N;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t m = i / N, n = i - m * N;
    const float* ar = a + m * K;
    const float* hr = w_hi + n * K;
    const float* lr = w_lo + n * K;
    float s = 0.0f;
    for (int64_t k = 0; k < K; k++) s = fmaf(ar[k], __fadd_rn(hr[k], lr[k]), s);  // hi + lo == w exactly
    if (bias) s = __fadd_rn(s, bias[n]);
    out[i] = s;
  }
}

// [rows, K] fp32 row-major, box = box_rows x 32 elements (128 bytes), 128-byte swizzle.
bool make_tmap_f32(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows,
                   std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 4};
  cuuint32_t box[2] = {(cuuint32_t)kFBlockK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(fp32 operand) failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

}  // namespace

int fgemm_setup(std::string* why) {
  cudaError_t e = cudaFuncSetAttribute(fgemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kFSmemBytes);
  if (e != cudaSuccess) {
    if (why) *why = std::string("cudaFuncSetAttribute(fp32 GEMM, max dynamic smem): ") + cudaGetErrorString(e);
    return SDQ_ERR_CUDA;
  }
  return SDQ_OK;
}

cudaError_t launch_transpose_split(const float* w_kn, int64_t K, int64_t N, float* hi_nk, float* lo_nk,
                                   cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32));
  count_launch();
  transpose_split_kernel<<<grid, 256, 0, s>>>(w_kn, K, N, hi_nk, lo_nk);
  return cudaGetLastError();
}

cudaError_t launch_fmatmul(const float* a, int64_t M, int64_t K, const float* w_hi, const float* w_lo,
                           int64_t N, const float* bias, float* out, float* a_hi, float* a_lo,
                           int* status, uint32_t flags, int sm_count, cudaStream_t s, std::string* why) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  const bool tc_ok = g_encode != nullptr && !(flags & SDQ_FORCE_SIMT) && K > 0 && K % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(a_hi) | reinterpret_cast<uintptr_t>(a_lo) |
                       reinterpret_cast<uintptr_t>(w_hi) | reinterpret_cast<uintptr_t>(w_lo)) & 15) == 0 &&
                     M < (int64_t(1) << 31) && N < (int64_t(1) << 31) && K < (int64_t(1) << 31);
  if (!tc_ok) {
    int64_t blocks = (M * N + 255) / 256;
    if (blocks > (int64_t)sm_count * 16) blocks = (int64_t)sm_count * 16;
    count_launch();
    fgemm_simt_kernel<<<(unsigned)blocks, 256, 0, s>>>(a, w_hi, w_lo, M, N, K, bias, out);
    return cudaGetLastError();
  }
  int64_t blocks = (M * K + 255) / 256;
  if (blocks > (int64_t)sm_count * 16) blocks = (int64_t)sm_count * 16;
  count_launch();
  split_tf32_kernel<<<(unsigned)blocks, 256, 0, s>>>(a, M * K, a_hi, a_lo);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo, tout;
  if (!make_tmap_f32(&ta_hi, a_hi, M, K, BLOCK_M, why) || !make_tmap_f32(&ta_lo, a_lo, M, K, BLOCK_M, why) ||
      !make_tmap_f32(&tb_hi, w_hi, N, K, kFBlockN, why) || !make_tmap_f32(&tb_lo, w_lo, N, K, kFBlockN, why))
    return cudaErrorInvalidValue;
  const int use_tma_store = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  if (use_tma_store) {
    if (!make_out_tmap(&tout, out, M, N, why)) return cudaErrorInvalidValue;
  } else {
    tout = ta_hi;  // unused by the kernel
  }
  FGemmArgs g;
  g.M = M; g.N = N; g.K = K; g.bias = bias; g.out = out; g.status = status;
  const int64_t tiles = ((M + BLOCK_M - 1) / BLOCK_M) * ((N + kFBlockN - 1) / kFBlockN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles < sm_count ? tiles : sm_count));
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = kFSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see grid_dependency_wait()
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, fgemm_tc_kernel, ta_hi, ta_lo, tb_hi, tb_lo, tout, use_tma_store, g);
}

}  // namespace sdq
