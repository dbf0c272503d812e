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
// Integer accumulation is exact and order-free, so any tiling -- and any split of K
// whose int32 partial sums are added afterwards -- gives the reference's sums bit for
// bit.  This file holds the 1-CTA kernel (small problems, odd N, accumulator dump,
// split-K) and the dispatch; the 2-CTA kernel for large problems is in
// qgemm_tcgen05_2cta.cu.
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
  // epilogue staging: per epilogue warp one 32x32 fp32 box (4 KiB) for the bulk tensor stores
  static constexpr int kStagingBytes = 8 * 4096;
  // stages + staging + barriers/bookkeeping + slack to realign the dynamic base to 1024 B
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
  // Split-K: a work item is (tile, K slice).  Slices of one tile add their int32 partial
  // sums into g.splitk_acc with bulk tensor reductions (integer addition: exact in any order); a second
  // kernel turns the sums into fp32.  k_splits == 1 is the ordinary case.
  const int k_splits = g.k_splits > 1 ? g.k_splits : 1;
  const int kb_per_split = (num_k_blocks + k_splits - 1) / k_splits;
  const int num_work = num_tiles * k_splits;

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
    if (use_tma_store || g.k_splits > 1) prefetch_tmap(&tmap_out);
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
      grid_dependency_wait();  // aq is written by the quantize kernel launched just before
      const uint64_t keep_policy = policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; ok && work < num_work; work += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(work % num_tiles, num_m_blocks, num_n_blocks, m_blk, n_blk);
        const int kb0 = (work / num_tiles) * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, num_k_blocks);
        for (int kb = kb0; kb < kb1; kb++) {
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
      for (int work = blockIdx.x; ok && work < num_work; work += gridDim.x) {
        ok = mbar_wait(bar_tempty + 8 * abuf, aphase ^ 1u, abort_flag, g.status, 0x200 | 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + abuf * BLOCK_N;
        const int kb0 = (work / num_tiles) * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, num_k_blocks);
        for (int kb = kb0; kb < kb1; kb++) {
          ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 0x200 | 2);
          if (!ok) break;
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_a + stage * C::kABytes);
          const uint64_t bdesc = make_smem_desc(smem_b + stage * C::kBBytes);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; k++) {
            // stepping K by 32 bytes inside the swizzle atom = +2 in the 16-byte address field
            umma_i8(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)),
                    bdesc + (uint64_t)(k * (UMMA_K >> 4)), C::kIdesc, (uint32_t)(((kb - kb0) | k) != 0));
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
    grid_dependency_wait();  // a_scale (and a split-K accumulator's memset) come from earlier work
    uint32_t abuf = 0, aphase = 0;
    bool ok = true;
    for (int work = blockIdx.x; ok && work < num_work; work += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(work % num_tiles, num_m_blocks, num_n_blocks, m_blk, n_blk);
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
          if (k_splits > 1) {
            // raw partial sums: staged like an output box, then added into the int32
            // accumulator by a bulk tensor reduction (tmap_out describes g.splitk_acc here)
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              st_shared_v4_b32(box + (uint32_t)(lane * 128 + (((j >> 2) ^ (lane & 7)) << 4)), r[j],
                               r[j + 1], r[j + 2], r[j + 3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_reduce_add_2d(&tmap_out, box, (int)nc, (int)row0);
              bulk_commit();
            }
          } else if (use_tma_store) {
            float o[32];
            switch (mode) {
              case 0: chunk_values<false, false>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
              case 1: chunk_values<true, false>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
              case 2: chunk_values<false, true>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
              default: chunk_values<true, true>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
            }
            float4 x[8];
            if (g.residual) chunk_load_residual(g.residual, row0, g.M, g.N, nc, lane, x);
            // The values go through a swizzled 32x32 fp32 box in shared memory; one bulk
            // tensor store then writes full 128-byte lines and clips rows >= M, columns >= N.
            if (lane == 0) bulk_wait_read<0>();  // the previous store has finished reading the box
            __syncwarp();
            if (g.residual) {  // x passes through the box so that each thread gets its own row
              chunk_stage_residual(box, lane, x);
              __syncwarp();
              chunk_apply_residual(box, lane, o, g.gate, nc, g.N);
            }
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
                float o = epilogue_value((int)r[j], a_s, __ldg(g.b_scale + nc + j),
                                         g.bias ? g.bias + nc + j : nullptr, gelu);
                if (g.residual)
                  o = residual_value(o, g.residual[row * g.N + nc + j], g.gate ? g.gate + nc + j : nullptr);
                out_row[nc + j] = o;
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

// Second step of split-K: fp32 outputs from the summed int32 accumulators.
__global__ void __launch_bounds__(256) splitk_finalize_kernel(GemmArgs g) {
  const bool gelu = (g.flags & SDQ_GELU_TANH) != 0;
  const int64_t total = g.M * g.N;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t row = i / g.N, col = i - row * g.N;
    const int acc = g.splitk_acc[i];
    if (g.acc_dump) g.acc_dump[i] = acc;
    float o = epilogue_value(acc, g.a_scale[row], __ldg(g.b_scale + col),
                             g.bias ? g.bias + col : nullptr, gelu);
    if (g.residual) o = residual_value(o, g.residual[i], g.gate ? g.gate + col : nullptr);
    g.out[i] = o;
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
                            g.acc_dump == nullptr && g.k_splits <= 1 &&
                            (reinterpret_cast<uintptr_t>(g.residual) & 15) == 0 &&
                            epilogue_vectors_aligned(g);
  if (g.k_splits > 1) {
    if (!make_out_tmap(&tout, g.splitk_acc, g.M, g.N, why, CU_TENSOR_MAP_DATA_TYPE_INT32))
      return cudaErrorInvalidValue;
  } else if (use_tma_store) {
    if (!make_out_tmap(&tout, g.out, g.M, g.N, why)) return cudaErrorInvalidValue;
  } else {
    tout = ta;  // unused by the kernel
  }
  const int64_t work = ((g.M + BLOCK_M - 1) / BLOCK_M) * ((g.N + BLOCK_N - 1) / BLOCK_N) *
                       (g.k_splits > 1 ? g.k_splits : 1);
  const unsigned grid = (unsigned)(work < sm_count ? work : sm_count);
  count_launch();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see grid_dependency_wait()
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, qgemm_tc_kernel<BLOCK_N>, ta, tb, tout, use_tma_store, g);
  if (e == cudaSuccess && g.k_splits > 1) {
    int64_t blocks = (g.M * g.N + 255) / 256;
    if (blocks > (int64_t)sm_count * 8) blocks = (int64_t)sm_count * 8;
    count_launch();
    splitk_finalize_kernel<<<(unsigned)blocks, 256, 0, s>>>(g);
    e = cudaGetLastError();
  }
  return e;
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

namespace {
// Small problems (too few tiles to give every SM pair a 256x256 tile) are bound by how
// fast the SMs can pull operand bytes, wave by wave.  Estimated time of a plan:
//   waves x (k-blocks per slice x max(stage bytes / per-SM fetch rate, MMA time) + fixed)
// plus the memset + finalize launches when K is split.  A narrow N tile spreads the
// weight bytes over more SMs but re-reads the activation tile once per column block; a
// K split multiplies the CTAs without re-reading anything.
struct Plan { int bn; int splits; };
Plan plan_small(const GemmArgs& g, int sm_count, bool allow_split) {
  const int64_t mb = (g.M + BLOCK_M - 1) / BLOCK_M;
  const int kb = (int)((g.K + BLOCK_K - 1) / BLOCK_K);
  const double rows_frac = (double)g.M / (double)(mb * BLOCK_M);  // rows past M are not fetched
  Plan best = {256, 1};
  double best_t = 1e30;
  for (int bn : {256, 128, 64, 32}) {
    for (int splits : {1, 2, 3, 4, 6, 8, 12, 16}) {
      if (splits > 1 && (!allow_split || kb / splits < 4 || g.N % 4 != 0)) continue;
      const int kbs = (kb + splits - 1) / splits;
      if (splits > 1 && (splits - 1) * kbs >= kb) continue;  // the last slice would be empty
      const int64_t work = mb * ((g.N + bn - 1) / bn) * splits;
      const double waves = (double)((work + sm_count - 1) / sm_count);
      const double stage_bytes = BLOCK_M * BLOCK_K * rows_frac + (double)bn * BLOCK_K;
      const double t_fetch = stage_bytes / 120e3;               // us at ~120 GB/s per SM
      const double t_mma = 4.0 * (bn / 256.0) * 128.0 / 1.9e3;  // us: 128 cycles per N=256 MMA
      double t = waves * (kbs * (t_fetch > t_mma ? t_fetch : t_mma) + 1.5 + 0.25 * bn / 32.0);
      if (splits > 1) t += 5.0 + (double)g.M * g.N * 4.0 * 3.0 / 3e6;  // memset + reductions + finalize
      if (t < best_t) { best_t = t; best = {bn, splits}; }
    }
  }
  return best;
}
}  // namespace

int qgemm_tc_plan_splits(const GemmArgs& g, int sm_count) {
  if (!qgemm_tc_supported(g) || qgemm_tc2_wanted(g, sm_count)) return 1;
  return plan_small(g, sm_count, true).splits;
}

cudaError_t launch_qgemm_tc(const GemmArgs& g, int sm_count, cudaStream_t s, std::string* why) {
  if (qgemm_tc2_wanted(g, sm_count)) return launch_qgemm_tc2(g, sm_count, s, why);
  GemmArgs a = g;
  Plan p;
  if (g.splitk_acc && g.k_splits > 1) {
    // the caller sized and cleared the accumulator for this many slices: honour it
    p = plan_small(g, sm_count, true);
    if (p.splits != g.k_splits) {
      p = plan_small(g, sm_count, false);
      p.splits = g.k_splits;
    }
  } else {
    p = plan_small(g, sm_count, false);
  }
  a.k_splits = p.splits;
  switch (p.bn) {
    case 256: return launch_t<256>(a, sm_count, s, why);
    case 128: return launch_t<128>(a, sm_count, s, why);
    case 64: return launch_t<64>(a, sm_count, s, why);
    default: return launch_t<32>(a, sm_count, s, why);
  }
}

}  // namespace sdq
