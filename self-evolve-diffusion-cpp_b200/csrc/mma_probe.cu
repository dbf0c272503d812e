// A measuring stick, not part of the data path: the rate at which one B200 retires
// tcgen05.mma kind::i8 instructions when nothing else limits them -- operands already in
// shared memory, no TMA, no epilogue, no global traffic.  Every SM issues M=128 x N=256 x K=32
// int8 MMAs back to back on a fixed pair of operand tiles.  The result is the ceiling the
// GEMM kernels of this library are compared with ("of measured int8 MMA peak"), taken on the
// same GPU, under the same power cap, by the same timing method.
#include "tc_common.cuh"

namespace sdq {
namespace {
using namespace tc;

constexpr int kProbeN = 256;
constexpr int kProbeThreads = 128;
constexpr int kProbeSmem = (BLOCK_M + kProbeN) * BLOCK_K + 1024 + 64;
constexpr uint32_t kProbeIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kProbeN >> 3) << 17) |
                                 ((uint32_t)(BLOCK_M >> 4) << 24);

__global__ void __launch_bounds__(kProbeThreads, 1) i8_mma_probe_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_a = base, smem_b = base + BLOCK_M * BLOCK_K;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (BLOCK_M + kProbeN) * BLOCK_K);
  const uint32_t bar = smem_u32(bars);  // two barriers, used alternately
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // operand bytes: a fixed pseudo-random pattern (all-zero operands would flatter the power draw)
  for (uint32_t i = threadIdx.x; i < (BLOCK_M + kProbeN) * BLOCK_K / 4; i += kProbeThreads)
    reinterpret_cast<uint32_t*>(smem)[i] = (i * 2654435761u) ^ (blockIdx.x * 40503u);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init(bar + 8, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> async proxy reads
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == 1 && lane == 0) {
    const uint64_t adesc = make_smem_desc(smem_a), bdesc = make_smem_desc(smem_b);
    uint32_t phase[2] = {0, 0};
    bool ok = true;
    // batches of 16 MMAs (4 k-blocks' worth), committed to alternating barriers; a batch is
    // issued only after the batch before the previous one has retired: two in flight
    for (int it = 0; ok && it < iters; it++) {
      const int b = it & 1;
      if (it >= 2) {
        ok = mbar_wait(bar + 8 * b, phase[b], abort_flag, status, 0x2100 | 1);
        phase[b] ^= 1u;
        tc_fence_after();
      }
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < 16; j++)
        umma_i8(tmem_base + b * kProbeN, adesc + (uint64_t)((j & 3) * 2), bdesc + (uint64_t)((j & 3) * 2),
                kProbeIdesc, (uint32_t)(j != 0));
      umma_commit(bar + 8 * b);
    }
    // drain: the last one or two batches
    for (int it = (iters >= 2 ? iters - 2 : 0); ok && it < iters; it++) {
      const int b = it & 1;
      ok = mbar_wait(bar + 8 * b, phase[b], abort_flag, status, 0x2100 | 2);
      phase[b] ^= 1u;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// Self-test of the time-out path: one warp waits on a barrier that nothing ever arrives on,
// through the same bounded wait the GEMM kernels use, with a limit of `limit_ns`.  The wait runs
// out, the status word receives the code, the abort flag is raised and the kernel returns: what
// a GEMM does when one of its waits gives up, without anything being stuck.
__global__ void __launch_bounds__(32, 1) wait_expiry_kernel(uint64_t limit_ns, int code, int* status,
                                                            int* outcome) {
  __shared__ __align__(8) uint64_t bar_mem;
  __shared__ int abort_word;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(bar, 0, &abort_word, status, code, limit_ns);
  __syncwarp();
  // every lane sees the flag the waiting lane raised, as the other roles of a GEMM CTA would
  if (threadIdx.x == 0) *outcome = (ok ? 1 : 0) | (*(volatile int*)&abort_word ? 2 : 0);
}

}  // namespace

int wait_expiry_selftest(int limit_ms, int code, int* status_dev, int* outcome_dev, cudaStream_t s) {
  count_launch();
  wait_expiry_kernel<<<1, 32, 0, s>>>((uint64_t)limit_ms * 1000000ull, code, status_dev, outcome_dev);
  SDQ_CUDA(cudaGetLastError());
  return SDQ_OK;
}

// Runs the probe on every SM; *seconds receives the device time of the launch.
int int8_mma_probe(int sm_count, int iters, int* status_dev, double* seconds, double* ops) {
  static bool attr_done = false;
  if (!attr_done) {
    SDQ_CUDA(cudaFuncSetAttribute(i8_mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem));
    attr_done = true;
  }
  cudaEvent_t e0, e1;
  SDQ_CUDA(cudaEventCreate(&e0));
  SDQ_CUDA(cudaEventCreate(&e1));
  SDQ_CUDA(cudaEventRecord(e0, 0));
  count_launch();
  i8_mma_probe_kernel<<<sm_count, kProbeThreads, kProbeSmem, 0>>>(iters, status_dev);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaEventRecord(e1, 0);
  if (e == cudaSuccess) e = cudaEventSynchronize(e1);
  float ms = 0;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  SDQ_CUDA(e);
  *seconds = ms * 1e-3;
  *ops = (double)sm_count * iters * 16.0 * 2.0 * BLOCK_M * kProbeN * UMMA_K;
  return SDQ_OK;
}

}  // namespace sdq
