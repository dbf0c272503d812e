// Shared pieces of the tcgen05 GEMM kernels: tile constants, inline-PTX wrappers
// (mbarrier, TMA, tcgen05), the shared-memory matrix descriptor, the tile order, the
// specialised epilogue arithmetic, and the host-side tensor-map encoders.
#pragma once
#include <cuda.h>

#include <string>

#include "epilogue.cuh"
#include "sdq_internal.h"

namespace sdq {
namespace tc {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;  // int8 elements = bytes: one 128-byte swizzle row
constexpr int UMMA_K = 32;    // K of one kind::i8 instruction
constexpr int kNumThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr uint32_t kTryWaitHintNs = 20000;  // upper bound on one hardware-suspended try_wait

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kTryWaitHintNs)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when it gave up (or another role already did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code, uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        __threadfence_system();
        return false;
      }
    }
  }
}

// The same bounded wait, polling without the hardware suspend: for a single lane whose wake-up
// latency sits on the critical path (an MMA issuer between dependent batches of instructions).
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int code) {
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 1023u) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        __threadfence_system();
        return false;
      }
    }
  }
}

// Programmatic dependent launch, consumer side: returns once every kernel this grid depends
// on in its stream has completed and its writes are visible.  Everything before it (barrier
// set-up, tensor-memory allocation, descriptor prefetch) may overlap the producer kernel.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Warp-wide bounded wait: lane 0 polls, the other lanes park at the shuffle (no issue
// slots, no power burnt spinning); every lane returns the same verdict.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile int* abort_flag, int* status, int code) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// Bulk tensor reduction: adds a 32x32 int32 box from shared memory into global memory
// (element-wise integer add performed by the memory system; clipped like a store).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::
                   "l"(reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void st_shared_v4_b32(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                                 uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}
// L2 eviction policies: weights are re-read by every band of row-blocks (keep them),
// outputs are written once and not read again by this kernel (let them go first).
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int x, int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// Bulk tensor store of a 32x32 fp32 box from shared memory; rows/columns outside the
// tensor are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, uint32_t src, int x, int y,
                                                  uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::
          "l"(reinterpret_cast<uint64_t>(map)),
      "r"(src), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, s8 x s8 -> s32.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t receives lane (base_lane+t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes,
// written by TMA with SWIZZLE_128B: 8-row groups are 1024 bytes apart (SBO),
// descriptor version 1 (Blackwell), layout type 2 (128-byte swizzle).  The
// leading-byte-offset field is not used by swizzled K-major layouts; it is set
// to 1 (16 bytes) as the canonical encoding does.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Tile order.  Consecutive tile indices (= the tiles the 148 CTAs work on at the same
// time) walk down a band of kGroupM row-blocks before moving to the next column-block,
// so a wave touches ~16 A tiles and ~9 B tiles instead of 3 and all of them: each
// operand tile is fetched from HBM once per band and then served to its other users
// from L2, and the weight matrix is re-read once per band rather than once per row-block.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords_g(int tile, int num_m_blocks, int num_n_blocks,
                                              int group_m, int& m_blk, int& n_blk) {
  const int per_group = group_m * num_n_blocks;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int gsize = min(group_m, num_m_blocks - first_m);
  const int r = tile - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}
__device__ __forceinline__ void tile_coords(int tile, int num_m_blocks, int num_n_blocks,
                                            int& m_blk, int& n_blk) {
  tile_coords_g(tile, num_m_blocks, num_n_blocks, kGroupM, m_blk, n_blk);
}

// 32 consecutive outputs of one row: rescale (+bias) (+GELU), compile-time specialised.
template <bool BIAS, bool GELU>
__device__ __forceinline__ void chunk_values(const uint32_t (&r)[32], float a_s,
                                             const float* __restrict__ b_scale,
                                             const float* __restrict__ bias, int64_t nc, int64_t N,
                                             float (&o)[32]) {
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    float4 bs = make_float4(0.f, 0.f, 0.f, 0.f), bb = bs;
    if (nc + j < N) {  // N % 4 == 0 on this path: a group of 4 is wholly inside or outside
      bs = __ldg(reinterpret_cast<const float4*>(b_scale + nc + j));
      if (BIAS) bb = __ldg(reinterpret_cast<const float4*>(bias + nc + j));
    }
    const float sc[4] = {bs.x, bs.y, bs.z, bs.w}, bi[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
    for (int t = 0; t < 4; t++) {
      float v = rescale((int)r[j + t], a_s, sc[t]);
      if (BIAS) v = __fadd_rn(v, bi[t]);
      if (GELU) v = gelu_tanh(v);
      o[j + t] = v;
    }
  }
}

// Residual epilogue, three steps around the staging box of a 32x32 chunk.
// (1) The warp fetches the chunk of x (the residual) with coalesced loads: one instruction
// covers four whole 128-byte rows, lane l taking 16-byte piece l%8 of row 4i + l/8.  Ordinary
// coherent loads: x may be the output buffer itself (the update is in place in the reference),
// and every element is read before the bulk store of the same chunk overwrites it.
__device__ __forceinline__ void chunk_load_residual(const float* __restrict__ res, int64_t row0,
                                                    int64_t M, int64_t N, int64_t nc, int lane,
                                                    float4 (&x)[8]) {
  const int64_t col = nc + (lane & 7) * 4;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int64_t row = row0 + i * 4 + (lane >> 3);
    x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < M && col < N) x[i] = *reinterpret_cast<const float4*>(res + row * N + col);
  }
}
// (2) The pieces go into the (free) staging box at the swizzled positions the output will take.
__device__ __forceinline__ void chunk_stage_residual(uint32_t box, int lane, const float4 (&x)[8]) {
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int r = i * 4 + (lane >> 3);
    st_shared_v4(box + (uint32_t)(r * 128 + (((lane & 7) ^ (r & 7)) << 4)), x[i]);
  }
}
// (3) Each thread reads its own row back (the same addresses its outputs are then written to)
// and applies o = x + o * gate[j] (one fused multiply-add), or x + o when there is no gate.
__device__ __forceinline__ void chunk_apply_residual(uint32_t box, int lane, float (&o)[32],
                                                     const float* __restrict__ gate, int64_t nc,
                                                     int64_t N) {
#pragma unroll
  for (int j = 0; j < 8; j++) {
    float4 xv;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(xv.x), "=f"(xv.y), "=f"(xv.z), "=f"(xv.w)
                 : "r"(box + (uint32_t)(lane * 128 + ((j ^ (lane & 7)) << 4))));
    const float xs[4] = {xv.x, xv.y, xv.z, xv.w};
    if (gate) {
      float4 gg = make_float4(0.f, 0.f, 0.f, 0.f);
      if (nc + 4 * j < N) gg = __ldg(reinterpret_cast<const float4*>(gate + nc + 4 * j));
      const float gs[4] = {gg.x, gg.y, gg.z, gg.w};
#pragma unroll
      for (int t = 0; t < 4; t++) o[4 * j + t] = fmaf(o[4 * j + t], gs[t], xs[t]);
    } else {
#pragma unroll
      for (int t = 0; t < 4; t++) o[4 * j + t] = __fadd_rn(xs[t], o[4 * j + t]);
    }
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
extern EncodeTiledFn g_encode;  // set by qgemm_tc_setup

// [rows, K] int8 row-major, box = box_rows x 128 bytes, 128-byte swizzle, zero fill outside.
inline bool make_tmap(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows,
               std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};  // bytes between rows
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

// out [M,N] fp32 row-major, box = 32 rows x 32 columns (128 bytes), 128-byte swizzle.
inline bool make_out_tmap(CUtensorMap* map, void* out, int64_t M, int64_t N, std::string* why,
                          CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32) {
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)N * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, dt, 2, out, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(out) failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

}  // namespace tc
}  // namespace sdq
