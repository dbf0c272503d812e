// int8 x int8 -> int32 GEMM on the Blackwell tensor cores (tcgen05, kind::i8)
// with the fp32 rescale / bias / GELU epilogue of the quantized linear.
//
//   acc[i,j] = sum_k aq[i,k] * bq[j,k]          (reference src/core/qgemm.cpp:22-59)
//   out[i,j] = (float)acc * (a_scale[i]*b_scale[j])   (src/core/qgemm.cpp:123-124,135)
//
// Both operands are K-major ("TN"): aq is [M,K] row-major, bq is the .sdcpp
// weight [N,K] row-major as stored in the file -- no repack.
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0, one lane : TMA producer.  Per k-block it loads a 128 x 128 B tile
//                      of aq and a BLOCK_N x 128 B tile of bq (SWIZZLE_128B)
//                      into a ring of shared-memory stages.
//   warp 1, one lane : MMA issuer.  4 x tcgen05.mma (M=128, N=BLOCK_N, K=32)
//                      per stage into one of two TMEM accumulator buffers;
//                      tcgen05.commit releases the stage / publishes the tile.
//   warps 2..9       : epilogue.  tcgen05.ld the finished accumulator (two warps
//                      per 32-lane TMEM quarter, alternate 32-column chunks),
//                      rescale, stage in shared memory, bulk tensor store.
//                      The second TMEM buffer lets tile t's epilogue overlap
//                      tile t+1's main loop.
// Integer accumulation is exact and order-free, so any tiling gives the
// reference's sums bit for bit.
//
// Every wait on an mbarrier is bounded: after ~2 s it records a code in the
// status word, raises a CTA-wide abort flag, and all roles fall through to the
// common exit, which frees the tensor memory.
#include <cstdio>

#include "tc_common.cuh"

namespace sdq {
namespace tc {
EncodeTiledFn g_encode = nullptr;
}
namespace {
using namespace tc;


template <int BLOCK_N>
struct Cfg {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kABytes = BLOCK_M * BLOCK_K;
  static constexpr int kBBytes = BLOCK_N * BLOCK_K;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BLOCK_N;  // two accumulator buffers; a power of two >= 32
  // stages + barriers/bookkeeping + slack to realign the dynamic base to 1024 B
  // epilogue staging: per epilogue warp one 32x32 fp32 box (4 KiB) for TMA stores
  static constexpr int kStagingBytes = 8 * 4096;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 256 + 1024;
  // instruction descriptor: D=s32 (2<<4), A=s8 (1<<7), B=s8 (1<<10), both K-major,
  // N>>3 at bit 17, M>>4 at bit 24
  static constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) |
                                     ((uint32_t)(BLOCK_N >> 3) << 17) |
                                     ((uint32_t)(BLOCK_M >> 4) << 24);
};

// ---------------------------------------------------------------- the kernel
template <int BLOCK_N>
__global__ void __launch_bounds__(kNumThreads, 1)
    qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out, int use_tma_store, GemmArgs g) {
  using C = Cfg<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  // SWIZZLE_128B atoms (8 rows x 128 B) must start on 1024-byte boundaries.
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t smem_a = base;
  const uint32_t smem_b = base + C::kStages * C::kABytes;
  const uint32_t smem_staging = base + C::kStages * C::kStageBytes;
  uint8_t* book = smem + C::kStages * C::kStageBytes + C::kStagingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(book);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m_blocks = (int)((g.M + BLOCK_M - 1) / BLOCK_M);
  const int num_n_blocks = (int)((g.N + BLOCK_N - 1) / BLOCK_N);
  const int num_k_blocks = (int)((g.K + BLOCK_K - 1) / BLOCK_K);
  const int num_tiles = num_m_blocks * num_n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; s++) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 8);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    if (use_tma_store) prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer
      const uint64_t keep_policy = policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, num_m_blocks, num_n_blocks, m_blk, n_blk);
        for (int kb = 0; kb < num_k_blocks; kb++) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x100 | 1);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, C::kStageBytes);
          tma_load_2d(smem_a + stage * C::kABytes, &tmap_a, full, kb * BLOCK_K, m_blk * BLOCK_M);
          tma_load_2d_hint(smem_b + stage * C::kBBytes, &tmap_b, full, kb * BLOCK_K,
                           n_blk * BLOCK_N, keep_policy);
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuer
      uint32_t stage = 0, phase = 0, abuf = 0, aphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        ok = mbar_wait(bar_tempty + 8 * abuf, aphase ^ 1u, abort_flag, g.status, 0x200 | 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + abuf * BLOCK_N;
        for (int kb = 0; kb < num_k_blocks; kb++) {
          ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 0x200 | 2);
          if (!ok) break;
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_a + stage * C::kABytes);
          const uint64_t bdesc = make_smem_desc(smem_b + stage * C::kBBytes);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; k++) {
            // stepping K by 32 bytes inside the swizzle atom = +2 in the 16-byte address field
            umma_i8(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)),
                    bdesc + (uint64_t)(k * (UMMA_K >> 4)), C::kIdesc, (uint32_t)((kb | k) != 0));
          }
          umma_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs have read it
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * abuf);  // accumulator complete
        abuf ^= 1u;
        if (abuf == 0) aphase ^= 1u;
      }
    }
  } else {
    // -------------------------------------------------- epilogue (8 warps)
    // Two warps share each TMEM lane quarter (a warp may only read lanes 32*(warp%4)..+31)
    // and take alternate 32-column chunks of the accumulator.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int mode = (g.bias ? 1 : 0) | ((g.flags & SDQ_GELU_TANH) ? 2 : 0);
    const uint32_t box = smem_staging + (uint32_t)((warp - 2) * 4096);
    const uint64_t stream_policy = policy_evict_first();
    uint32_t abuf = 0, aphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, num_m_blocks, num_n_blocks, m_blk, n_blk);
      ok = mbar_wait_warp(bar_tfull + 8 * abuf, aphase, abort_flag, g.status, 0x300 | 1);
      if (!ok) break;
      tc_fence_after();
      const int64_t row0 = (int64_t)m_blk * BLOCK_M + quarter * 32;
      const int64_t row = row0 + lane;
      const bool row_ok = row < g.M;
      const float a_s = row_ok ? g.a_scale[row] : 0.0f;
      const int64_t n0 = (int64_t)n_blk * BLOCK_N;
      if (row0 < g.M) {  // warp-uniform: this warp's 32 rows are not all past the end
#pragma unroll 1
        for (int c = half; c < BLOCK_N / 32; c += 2) {
          const int64_t nc = n0 + c * 32;
          if (nc >= g.N) break;  // warp-uniform
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + abuf * BLOCK_N + c * 32 + ((uint32_t)(quarter * 32) << 16), r);
          tmem_ld_wait();
          if (use_tma_store) {
            float o[32];
            switch (mode) {
              case 0: chunk_values<false, false>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
              case 1: chunk_values<true, false>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
              case 2: chunk_values<false, true>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
              default: chunk_values<true, true>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
            }
            // The values go through a swizzled 32x32 fp32 box in shared memory; one bulk
            // tensor store then writes full 128-byte lines and clips rows >= M, columns >= N.
            if (lane == 0) bulk_wait_read<0>();  // the previous store has finished reading the box
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; j += 4)  // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
              st_shared_v4(box + (uint32_t)(lane * 128 + (((j >> 2) ^ (lane & 7)) << 4)),
                           make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]));
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d_hint(&tmap_out, box, (int)nc, (int)row0, stream_policy);
              bulk_commit();
            }
          } else if (row_ok) {
            // per-thread stores: odd N, unaligned out, or the accumulator dump is wanted
            float* out_row = g.out + row * g.N;
            int32_t* dump_row = g.acc_dump ? g.acc_dump + row * g.N : nullptr;
            const bool gelu = (mode & 2) != 0;
#pragma unroll
            for (int j = 0; j < 32; j++) {
              if (nc + j < g.N) {
                out_row[nc + j] = epilogue_value((int)r[j], a_s, __ldg(g.b_scale + nc + j),
                                                 g.bias ? g.bias + nc + j : nullptr, gelu);
                if (dump_row) dump_row[nc + j] = (int)r[j];
              }
            }
          }
        }
      }
      // hand the accumulator buffer back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * abuf);
      abuf ^= 1u;
      if (abuf == 0) aphase ^= 1u;
    }
  }

  // ---------------------------------------------------- common exit
  if (warp >= 2 && lane == 0) bulk_wait_read<0>();  // staged boxes fully read by the stores
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    // give bulk copies that may still be in flight time to land before the CTA's
    // shared memory is released (bounded: ~1 ms)
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();  // the dealloc is a warp-wide (.sync.aligned) instruction
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------- host side

template <int BLOCK_N>
cudaError_t launch_t(const GemmArgs& g, int sm_count, cudaStream_t s, std::string* why) {
  using C = Cfg<BLOCK_N>;
  CUtensorMap ta, tb, tout;
  if (!make_tmap(&ta, g.aq, g.M, g.K, BLOCK_M, why)) return cudaErrorInvalidValue;
  if (!make_tmap(&tb, g.bq, g.N, g.K, BLOCK_N, why)) return cudaErrorInvalidValue;
  // Bulk tensor stores need a 16-byte aligned base and row pitch; the accumulator dump
  // (a debugging aid) and odd N keep the per-thread store path.
  const int use_tma_store = (g.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(g.out) & 15) == 0) &&
                            g.acc_dump == nullptr;
  if (use_tma_store) {
    if (!make_out_tmap(&tout, g.out, g.M, g.N, why)) return cudaErrorInvalidValue;
  } else {
    tout = ta;  // unused by the kernel
  }
  const int64_t tiles = ((g.M + BLOCK_M - 1) / BLOCK_M) * ((g.N + BLOCK_N - 1) / BLOCK_N);
  const unsigned grid = (unsigned)(tiles < sm_count ? tiles : sm_count);
  count_launch();
  qgemm_tc_kernel<BLOCK_N><<<grid, kNumThreads, C::kSmemBytes, s>>>(ta, tb, tout, use_tma_store, g);
  return cudaGetLastError();
}

template <int BLOCK_N>
cudaError_t set_smem_attr() {
  return cudaFuncSetAttribute(qgemm_tc_kernel<BLOCK_N>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              Cfg<BLOCK_N>::kSmemBytes);
}

}  // namespace

int qgemm_tc_setup(std::string* why) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    if (why) *why = "cuTensorMapEncodeTiled is not available from this driver";
    return SDQ_ERR_CUDA;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  cudaError_t a = set_smem_attr<256>();
  if (a == cudaSuccess) a = set_smem_attr<128>();
  if (a == cudaSuccess) a = set_smem_attr<64>();
  if (a == cudaSuccess) a = set_smem_attr<32>();
  if (a != cudaSuccess) {
    if (why) *why = std::string("cudaFuncSetAttribute(max dynamic smem): ") + cudaGetErrorString(a);
    return SDQ_ERR_CUDA;
  }
  return qgemm_tc2_setup(why);
}

bool qgemm_tc_supported(const GemmArgs& g) {
  return g_encode != nullptr && g.M > 0 && g.N > 0 && g.K > 0 && (g.K % 16 == 0) &&
         ((reinterpret_cast<uintptr_t>(g.aq) & 15) == 0) &&
         ((reinterpret_cast<uintptr_t>(g.bq) & 15) == 0) && g.M < (int64_t(1) << 31) &&
         g.N < (int64_t(1) << 31) && g.K < (int64_t(1) << 31) &&
         ((g.M + BLOCK_M - 1) / BLOCK_M) * ((g.N + 31) / 32) < (int64_t(1) << 31);
}

cudaError_t launch_qgemm_tc(const GemmArgs& g, int sm_count, cudaStream_t s, std::string* why) {
  // Largest N tile that still gives every SM a tile; small problems take narrower
  // tiles so that more SMs pull weight bytes from HBM at once.
  if (qgemm_tc2_wanted(g, sm_count)) return launch_qgemm_tc2(g, sm_count, s, why);
  const int64_t mb = (g.M + BLOCK_M - 1) / BLOCK_M;
  auto tiles = [&](int bn) { return mb * ((g.N + bn - 1) / bn); };
  if (tiles(256) >= sm_count) return launch_t<256>(g, sm_count, s, why);
  if (tiles(128) >= sm_count) return launch_t<128>(g, sm_count, s, why);
  if (tiles(64) >= sm_count) return launch_t<64>(g, sm_count, s, why);
  return launch_t<32>(g, sm_count, s, why);
}

}  // namespace sdq
