// The large-problem variant of the tcgen05 int8 GEMM: two CTAs on neighbouring SMs
// (a cluster of 2) work on one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Per k-block each CTA stages only its own 128 rows of aq and its own 128 of the
// tile's 256 weight rows (32 KiB instead of 48 KiB), and the tensor cores of both SMs
// read the weight halves from both shared memories.  That cuts the L2->SM and the
// shared-memory traffic per MMA by a third and leaves room for 6 pipeline stages,
// which is what the 1-CTA kernel is short of at the int8 rate.
//
//   CTA rank r of the pair:  rows  m_pair*256 + r*128 .. +127   (its A half, its D rows)
//                            weight rows n_blk*256 + r*128 .. +127 (its B half)
//   leader (rank 0), one lane: issues every MMA; tcgen05.commit with a 2-CTA multicast
//                            releases a stage / publishes the accumulator in both CTAs
//   both CTAs' TMA lanes   : complete_tx on the LEADER's "full" barrier
//   both CTAs' epilogue    : read their own TMEM (128 lanes x 256 columns), store their
//                            own 128 rows, arrive on the LEADER's "tmem empty" barrier
// No TMA multicast is used.  Every wait is bounded as in the 1-CTA kernel, and the two
// CTAs leave through a cluster barrier so that neither frees shared or tensor memory
// the other may still signal.
//
// Last, partial wave.  With T tiles on C CTA pairs, the first floor(T/C) rounds give every
// pair a whole tile.  The remaining T mod C tiles would keep only some pairs busy for a
// whole tile time, so (when a scratch accumulator is supplied and it pays) their k-blocks are
// shared out instead: the tail's (T mod C) * KB k-block units are cut into C equal contiguous
// ranges, a pair runs its range (at most two segments, each a k-range of one tile) and adds the
// raw int32 partial sums into the scratch with bulk tensor reductions -- integer addition,
// exact in any order -- and tail_finalize_kernel then turns the sums of those tiles into
// fp32 outputs and clears the scratch for the next launch.
#include <cstdio>
#include <cstdlib>

#include "tc_common.cuh"

namespace sdq {
namespace {
using namespace tc;

constexpr int kBlockN2 = 256;
constexpr int kHalfBytes = BLOCK_M * BLOCK_K;         // 16 KiB: 128 rows x 128 B
constexpr int kTmemCols2 = 2 * kBlockN2;
// dynamic shared memory: pipeline stages + epilogue staging boxes + barriers + realignment slack
constexpr int smem_bytes2(int stages, int boxes, int a_copies = 1) {
  return stages * (a_copies * kHalfBytes + kHalfBytes) + 8 * 4096 * boxes + 256 + 1024;
}
// D=s32, A=B=s8, K-major both, N=256 (>>3 at bit 17), M=256 (>>4 at bit 24)
constexpr uint32_t kIdesc2 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlockN2 >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster-wide shared window, of CTA `rank`'s copy of a shared variable.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// 2-CTA form of the tiled load: the destination is this CTA's shared memory, the
// mbarrier may live in the partner CTA (cluster-window address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once
// the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}

// The work of one CTA pair: `rounds` whole tiles (tile = round * C + cluster), then the
// segments of its share of the tail.  Every role walks the same list.
struct Work {
  int tile;      // index into the tile order
  int kb0, kb1;  // k-block range
  int partial;   // 1: a tail segment, partial sums go to the scratch accumulator
};
struct WorkList {
  int rounds, first_tail, num_tiles, num_clusters, cluster_id, kblocks;
  int u0, u1;  // this pair's range of tail units (tile-major, k-block-minor)
  __device__ WorkList(int tiles, int clusters, int cluster, int kb, bool share_tail)
      : num_tiles(tiles), num_clusters(clusters), cluster_id(cluster), kblocks(kb) {
    rounds = share_tail ? tiles / clusters : (tiles + clusters - 1) / clusters;
    first_tail = rounds * clusters;
    const int64_t units = share_tail ? (int64_t)(tiles - first_tail) * kb : 0;
    u0 = (int)(units * cluster / clusters);
    u1 = (int)(units * (cluster + 1) / clusters);
  }
  __device__ bool get(int idx, Work& w) const {
    if (idx < rounds) {
      w.tile = idx * num_clusters + cluster_id;
      w.kb0 = 0; w.kb1 = kblocks; w.partial = 0;
      return w.tile < num_tiles;
    }
    if (u1 <= u0) return false;
    const int t = u0 / kblocks;  // first tail tile this pair touches
    const int seg = idx - rounds;
    if (seg == 0) {
      w.tile = first_tail + t;
      w.kb0 = u0 - t * kblocks;
      w.kb1 = min(kblocks, w.kb0 + (u1 - u0));
      w.partial = 1;
      return true;
    }
    if (seg == 1 && u1 > (t + 1) * kblocks) {
      w.tile = first_tail + t + 1;
      w.kb0 = 0;
      w.kb1 = u1 - (t + 1) * kblocks;
      w.partial = 1;
      return true;
    }
    return false;
  }
};

// Output tensor maps: one in the ordinary case; in the column-split multi-GPU form one per
// destination buffer (this GPU's and each peer's), all describing [M, out_ld] fp32.
struct OutMaps {
  CUtensorMap m[8];
};

// kStages2: depth of the operand ring; kBoxes: staging boxes per epilogue warp (with two, a
// warp fills one box while the bulk store of the other is still reading shared memory).
// kACopies > 1 is a measuring variant, not a product path: every k-block's A tile is fetched
// kACopies times into that many slots of the stage (the MMAs read the first).  With 4 copies a
// stage carries the bytes an fp32 A tile would -- what a GEMM that quantized its activations in
// its own prologue would have to move through shared memory -- at the ring depth that then still
// fits (2 stages of 80 KiB); the conversion itself (another shared-memory round trip per tile)
// is not even included.  Results are unchanged; only the time is of interest.
template <int kStages2, int kBoxes, bool kResidual, int kACopies = 1>
__global__ void __launch_bounds__(kNumThreads, 1)
    qgemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ OutMaps outs, int num_outs,
                     const __grid_constant__ CUtensorMap tmap_tail, GemmArgs g) {
  constexpr int kStagingBytes2 = 8 * 4096 * kBoxes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // same offset in both CTAs of the pair
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t smem_a = base;
  constexpr int kAStage = kACopies * kHalfBytes;       // bytes of A per stage
  constexpr int kStageBytes = kAStage + kHalfBytes;    // per CTA: A half (x copies) + B half
  const uint32_t smem_b = base + kStages2 * kAStage;
  const uint32_t smem_staging = base + kStages2 * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages2 * kStageBytes + kStagingBytes2);
  const uint32_t bar_full = smem_u32(bars);            // used in the leader only
  const uint32_t bar_empty = bar_full + 8 * kStages2;  // one per CTA, signalled by multicast commit
  const uint32_t bar_tfull = bar_empty + 8 * kStages2; // one per CTA, multicast commit
  const uint32_t bar_tempty = bar_tfull + 16;          // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;
  const int num_m_pairs = (int)((g.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M));
  const int num_n_blocks = (int)((g.N + kBlockN2 - 1) / kBlockN2);
  const int num_k_blocks = (int)((g.K + BLOCK_K - 1) / BLOCK_K);
  const int num_tiles = num_m_pairs * num_n_blocks;
  const int group_pairs = g.group_pairs > 0 ? g.group_pairs : kGroupM / 2;
  const WorkList work(num_tiles, num_clusters, cluster_id, num_k_blocks, g.tail_acc != nullptr);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; s++) {
      mbar_init(bar_full + 8 * s, 1);   // the leader's producer arrives once (+ both CTAs' bytes)
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 16);  // 8 epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int i = 0; i < num_outs; i++) prefetch_tmap(&outs.m[i]);
    if (g.tail_acc) prefetch_tmap(&tmap_tail);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols2);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer (both CTAs)
      grid_dependency_wait();  // aq is written by the quantize kernel launched just before
      const uint64_t keep_policy = policy_evict_last();
      const uint64_t a_policy = g.a_policy == 1 ? policy_evict_first()
                                : (g.a_policy == 2 ? keep_policy : policy_evict_normal());
      const uint64_t b_policy = g.b_policy == 1 ? policy_evict_normal() : keep_policy;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      Work w;
      for (int idx = 0; ok && work.get(idx, w); idx++) {
        int m_pair, n_blk;
        tile_coords_g(w.tile, num_m_pairs, num_n_blocks, group_pairs, m_pair, n_blk);
        const int row0 = (m_pair * 2 + (int)rank) * BLOCK_M;
        const int wrow0 = n_blk * kBlockN2 + (int)rank * BLOCK_M;
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x1100 | 1);
          if (!ok) break;
          const uint32_t full_leader = map_to_cta(bar_full + 8 * stage, 0);
          if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * kStageBytes);
#pragma unroll
          for (int copy = 0; copy < kACopies; copy++)
            tma_load_2d_pair(smem_a + stage * kAStage + copy * kHalfBytes, &tmap_a, full_leader,
                             kb * BLOCK_K, row0, a_policy);
          tma_load_2d_pair(smem_b + stage * kHalfBytes, &tmap_b, full_leader, kb * BLOCK_K, wrow0,
                           b_policy);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------------------------------ MMA issuer (leader CTA only)
      uint32_t stage = 0, phase = 0, abuf = 0, aphase = 0;
      bool ok = true;
      Work w;
      for (int idx = 0; ok && work.get(idx, w); idx++) {
        ok = mbar_wait(bar_tempty + 8 * abuf, aphase ^ 1u, abort_flag, g.status, 0x1200 | 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + abuf * kBlockN2;
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 0x1200 | 2);
          if (!ok) break;
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_a + stage * kAStage);
          const uint64_t bdesc = make_smem_desc(smem_b + stage * kHalfBytes);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; k++)
            umma_i8_pair(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)),
                         bdesc + (uint64_t)(k * (UMMA_K >> 4)), kIdesc2,
                         (uint32_t)(((kb - w.kb0) | k) != 0));
          umma_commit_pair(bar_empty + 8 * stage);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(bar_tfull + 8 * abuf);
        abuf ^= 1u;
        if (abuf == 0) aphase ^= 1u;
      }
    }
  } else {
    // -------------------------------------------------- epilogue (8 warps, both CTAs)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int mode = (g.bias ? 1 : 0) | ((g.flags & SDQ_GELU_TANH) ? 2 : 0);
    const uint32_t box0 = smem_staging + (uint32_t)((warp - 2) * 4096 * kBoxes);
    uint32_t box_sel = 0;
    const uint64_t stream_policy = policy_evict_first();
    const uint32_t tempty_leader0 = map_to_cta(bar_tempty, 0);
    grid_dependency_wait();  // a_scale comes from the quantize kernel
    uint32_t abuf = 0, aphase = 0;
    bool ok = true;
    Work w;
    for (int idx = 0; ok && work.get(idx, w); idx++) {
      int m_pair, n_blk;
      tile_coords_g(w.tile, num_m_pairs, num_n_blocks, group_pairs, m_pair, n_blk);
      ok = mbar_wait_warp(bar_tfull + 8 * abuf, aphase, abort_flag, g.status, 0x1300 | 1);
      if (!ok) break;
      tc_fence_after();
      const int64_t row0 = (int64_t)(m_pair * 2 + (int)rank) * BLOCK_M + quarter * 32;
      const int64_t row = row0 + lane;
      const float a_s = row < g.M ? g.a_scale[row] : 0.0f;
      const int64_t n0 = (int64_t)n_blk * kBlockN2;
      if (row0 < g.M) {
#pragma unroll 1
        for (int c = half; c < kBlockN2 / 32; c += 2) {
          const int64_t nc = n0 + c * 32;
          if (nc >= g.N) break;
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + abuf * kBlockN2 + c * 32 + ((uint32_t)(quarter * 32) << 16), r);
          if (w.partial) {
            // a tail segment: the raw partial sums are added into the scratch accumulator
            // (row = tail tile * 256 + row inside the tile, column = column inside the tile)
            tmem_ld_wait();
            const uint32_t box = box0 + box_sel * 4096;
            if (kBoxes > 1) box_sel ^= 1u;
            if (lane == 0) bulk_wait_read<kBoxes - 1>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              st_shared_v4_b32(box + (uint32_t)(lane * 128 + (((j >> 2) ^ (lane & 7)) << 4)), r[j],
                               r[j + 1], r[j + 2], r[j + 3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_reduce_add_2d(&tmap_tail, box, c * 32,
                                (w.tile - work.first_tail) * (2 * BLOCK_M) + (int)rank * BLOCK_M + quarter * 32);
              bulk_commit();
            }
            continue;
          }
          float4 x[8];
          if (kResidual)  // in flight while the accumulators arrive from tensor memory
            chunk_load_residual(g.residual, row0, g.M, g.N, nc, lane, x);
          tmem_ld_wait();
          float o[32];
          switch (mode) {
            case 0: chunk_values<false, false>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
            case 1: chunk_values<true, false>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
            case 2: chunk_values<false, true>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
            default: chunk_values<true, true>(r, a_s, g.b_scale, g.bias, nc, g.N, o); break;
          }
          const uint32_t box = box0 + box_sel * 4096;
          if (kBoxes > 1) box_sel ^= 1u;
          // the store that last read this box must have finished reading it
          if (lane == 0) bulk_wait_read<kBoxes - 1>();
          __syncwarp();
          if (kResidual) {  // x passes through the box so that each thread gets its own row
            chunk_stage_residual(box, lane, x);
            __syncwarp();
            chunk_apply_residual(box, lane, o, g.gate, nc, g.N);
          }
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            st_shared_v4(box + (uint32_t)(lane * 128 + (((j >> 2) ^ (lane & 7)) << 4)),
                         make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]));
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            // one staged box, one bulk store per destination (peer stores cross NVLink)
            for (int i = 0; i < num_outs; i++)
              tma_store_2d_hint(&outs.m[i], box, (int)(g.out_col0 + nc), (int)row0, stream_policy);
            bulk_commit();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * abuf);
      abuf ^= 1u;
      if (abuf == 0) aphase ^= 1u;
    }
  }

  // ---------------------------------------------------- common exit
  if (warp >= 2 && lane == 0) bulk_wait_read<0>();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);  // let bulk copies in flight land (~1 ms)
    __syncthreads();
  }
  // Neither CTA may release its shared / tensor memory while the partner can still signal it.
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, kTmemCols2);
  }
}

// Second step for the tiles of a shared last wave: fp32 outputs from the summed int32
// partial sums, which are cleared on the way so that the scratch is all zero again.
// grid = (tail tiles, 64): one group of 4 consecutive columns per thread, so that the pass is
// one round of independent 16-byte loads and stores (it sits between two dependent launches).
template <bool kResidual>
__global__ void __launch_bounds__(256) tail_finalize_kernel(GemmArgs g, int first_tail, int group_pairs) {
  const int num_m_pairs = (int)((g.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M));
  const int num_n_blocks = (int)((g.N + kBlockN2 - 1) / kBlockN2);
  int m_pair, n_blk;
  tile_coords_g(first_tail + (int)blockIdx.x, num_m_pairs, num_n_blocks, group_pairs, m_pair, n_blk);
  const bool gelu = (g.flags & SDQ_GELU_TANH) != 0;
  int4* acc = reinterpret_cast<int4*>(g.tail_acc + (size_t)blockIdx.x * (2 * BLOCK_M) * kBlockN2);
  constexpr int kVecs = 2 * BLOCK_M * kBlockN2 / 4;  // 16384 groups of 4 columns per tile
  for (int v = (int)blockIdx.y * 256 + (int)threadIdx.x; v < kVecs; v += (int)gridDim.y * 256) {
    const int r = v / (kBlockN2 / 4), c4 = (v - r * (kBlockN2 / 4)) * 4;
    const int64_t row = (int64_t)m_pair * (2 * BLOCK_M) + r, col = (int64_t)n_blk * kBlockN2 + c4;
    if (row >= g.M || col >= g.N) continue;  // never written: still zero
    const int4 a = acc[v];
    acc[v] = make_int4(0, 0, 0, 0);
    const float a_s = g.a_scale[row];
    const float4 bs = __ldg(reinterpret_cast<const float4*>(g.b_scale + col));
    float4 bb = make_float4(0.f, 0.f, 0.f, 0.f), gg = bb, xx = bb;
    if (g.bias) bb = __ldg(reinterpret_cast<const float4*>(g.bias + col));
    float* dst = g.out + row * g.N + col;
    if (kResidual) {
      xx = *reinterpret_cast<const float4*>(g.residual + row * g.N + col);
      if (g.gate) gg = __ldg(reinterpret_cast<const float4*>(g.gate + col));
    }
    const int av[4] = {a.x, a.y, a.z, a.w};
    const float sc[4] = {bs.x, bs.y, bs.z, bs.w}, bi[4] = {bb.x, bb.y, bb.z, bb.w};
    const float gs[4] = {gg.x, gg.y, gg.z, gg.w}, xs[4] = {xx.x, xx.y, xx.z, xx.w};
    float o[4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
      o[t] = epilogue_value(av[t], a_s, sc[t], g.bias ? &bi[t] : nullptr, gelu);
      if (kResidual) o[t] = residual_value(o[t], xs[t], g.gate ? &gs[t] : nullptr);
    }
    *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

// ---------------------------------------------------------------- host side
// 6 stages + 1 box and 5 stages + 2 boxes both fill the 227 KiB of an SM.
int tc2_config() {
  static const int cfg = [] {
    const char* v = getenv("SDQ_TC2_CONFIG");  // "61": 6 stages, 1 box; "52": 5 stages, 2 boxes
    return v ? atoi(v) : 61;
  }();
  return cfg == 52 ? 52 : 61;
}
namespace {
int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
}
// Tiles of the last, partial wave whose k-blocks are shared out, or 0 when every tile is
// left to one pair.  Sharing saves (1 - tail/C) of a tile time (~0.4 us per 128-byte
// k-block at the sustained int8 rate) and costs one more launch plus a pass over the
// scratch (~0.2 us per tile).
int plan_tail(const GemmArgs& g, int64_t tiles, int64_t clusters) {
  const int mode = env_int("SDQ_TC2_TAIL", 1);  // 0: never, 1: when it pays, 2: whenever possible
  if (mode == 0 || g.out_copies > 0) return 0;
  const int64_t tail = tiles % clusters;
  if (tail == 0) return 0;
  if (mode == 2) return (int)tail;
  const double kblocks = (double)((g.K + BLOCK_K - 1) / BLOCK_K);
  const double saved_us = (1.0 - (double)tail / (double)clusters) * kblocks * 0.40 - (4.0 + 0.2 * (double)tail);
  return saved_us > 1.0 ? (int)tail : 0;
}
// Height of a band of the tile walk, in 256-row pairs.  The 74 tiles in flight cover
// (band height) row pairs x (74 / band height) column blocks.  A band's rows of aq are fetched
// from HBM once if the band stays in L2 while its column blocks pass (otherwise once per wave),
// and the weight matrix is re-read once per band: so the band is made as tall as ~32 MB of aq
// allow, and no taller than 24 pairs.  Measured on the 720p FFN shapes (alternating loops):
// K = 3072: 12..30 pairs within 2 % of each other and 4..8 or 54 pairs 5-8 % slower, DRAM reads
// per launch 688 MB at 8 pairs, 365 MB at 24; K = 14336: all of 6..24 within 2 %, DRAM reads
// 1.35 GB at 8 pairs (29 MB of aq per band) against 1.93 GB at 24 (88 MB: re-read every wave).
int plan_group(const GemmArgs& g) {
  const int forced = env_int("SDQ_TC2_GROUP", 0);
  if (forced > 0) return forced;
  const int pairs = (int)(32.0e6 / (2.0 * BLOCK_M * (double)g.K));
  return pairs < 4 ? 4 : (pairs > 24 ? 24 : pairs);
}
}  // namespace

int qgemm_tc2_setup(std::string* why) {
  cudaError_t a = cudaSuccess;
  cudaFuncSetAttribute((const void*)qgemm_tc2_kernel<2, 1, false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       smem_bytes2(2, 1, 4));
  cudaFuncSetAttribute((const void*)qgemm_tc2_kernel<2, 1, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       smem_bytes2(2, 1, 1));
  const void* kernels[4] = {(const void*)qgemm_tc2_kernel<6, 1, false>, (const void*)qgemm_tc2_kernel<6, 1, true>,
                            (const void*)qgemm_tc2_kernel<5, 2, false>, (const void*)qgemm_tc2_kernel<5, 2, true>};
  for (int i = 0; i < 4 && a == cudaSuccess; i++)
    a = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize,
                             i < 2 ? smem_bytes2(6, 1) : smem_bytes2(5, 2));
  if (a != cudaSuccess) {
    if (why) *why = std::string("cudaFuncSetAttribute(2-CTA GEMM, max dynamic smem): ") + cudaGetErrorString(a);
    return SDQ_ERR_CUDA;
  }
  return SDQ_OK;
}

// The pair kernel stores only through bulk tensor stores and its epilogue reads the scales,
// bias and gate four floats at a time: N % 4 == 0, 16-byte aligned out / residual / b_scale /
// bias / gate, no accumulator dump.
const char* qgemm_tc2_unfit(const GemmArgs& g) {
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (g.acc_dump) return "the accumulator dump needs the 1-CTA kernel";
  if (misaligned(g.b_scale)) return "the weight scales are not 16-byte aligned";
  if (g.bias && misaligned(g.bias)) return "the bias is not 16-byte aligned";
  if (g.residual && g.gate && misaligned(g.gate)) return "the gate is not 16-byte aligned";
  if (g.residual && misaligned(g.residual)) return "the residual is not 16-byte aligned";
  if (g.out_copies > 0) {
    if (g.residual) return "the column-split form has no residual epilogue";
    if (g.out_ld % 4 != 0 || g.out_col0 % 4 != 0) return "the row pitch or column offset of the destinations is not a multiple of 4";
    for (int i = 0; i < g.out_copies; i++)
      if (misaligned(g.out_all[i])) return "a destination is not 16-byte aligned";
    return nullptr;
  }
  if (g.N % 4 != 0) return "N is not a multiple of 4";
  if (misaligned(g.out)) return "out is not 16-byte aligned";
  return nullptr;
}

// Tiles of the last wave the launcher would share out if it is given a scratch accumulator
// (GemmArgs::tail_acc) of at least that many tiles; 0: it needs none.
int qgemm_tc2_tail_tiles(const GemmArgs& g, int sm_count) {
  const int64_t tiles = ((g.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) * ((g.N + kBlockN2 - 1) / kBlockN2);
  return plan_tail(g, tiles, sm_count / 2);
}

// ... and it pays off once every cluster has at least one tile.
bool qgemm_tc2_wanted(const GemmArgs& g, int sm_count) {
  static const int forced = env_int("SDQ_TC_VARIANT", 0);  // "1": never, "2": whenever possible
  if (qgemm_tc2_unfit(g)) return false;
  if (g.out_copies > 0) return true;  // the caller asked for the fused form; it has no other kernel
  if (forced == 1) return false;
  const int64_t tiles = ((g.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) * ((g.N + kBlockN2 - 1) / kBlockN2);
  if (forced == 2) return true;
  return tiles >= sm_count / 2;
}

cudaError_t launch_qgemm_tc2(const GemmArgs& g_in, int sm_count, cudaStream_t s, std::string* why) {
  GemmArgs g = g_in;
  CUtensorMap ta, tb, ttail;
  OutMaps outs;
  if (!make_tmap(&ta, g.aq, g.M, g.K, BLOCK_M, why)) return cudaErrorInvalidValue;
  if (!make_tmap(&tb, g.bq, g.N, g.K, BLOCK_M, why)) return cudaErrorInvalidValue;  // 128-row halves
  int num_outs = 1;
  if (g.out_copies > 0) {
    num_outs = g.out_copies;
    for (int i = 0; i < num_outs; i++)
      if (!make_out_tmap(&outs.m[i], g.out_all[i], g.M, g.out_ld, why)) return cudaErrorInvalidValue;
  } else {
    if (!make_out_tmap(&outs.m[0], g.out, g.M, g.N, why)) return cudaErrorInvalidValue;
  }
  for (int i = num_outs; i < 8; i++) outs.m[i] = outs.m[0];
  const int64_t tiles = ((g.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) * ((g.N + kBlockN2 - 1) / kBlockN2);
  int64_t clusters = sm_count / 2;
  int tail = plan_tail(g, tiles, clusters);
  if (!g.tail_acc || tail > g.tail_cap_tiles) tail = 0;
  if (tail > 0) {
    // [tail tiles x 256 rows, 256 columns] int32, boxes of 32 x 32 like the output
    if (!make_out_tmap(&ttail, g.tail_acc, (int64_t)tail * 2 * BLOCK_M, kBlockN2, why, CU_TENSOR_MAP_DATA_TYPE_INT32))
      return cudaErrorInvalidValue;
  } else {
    g.tail_acc = nullptr;
    ttail = ta;  // unused by the kernel
    if (tiles < clusters) clusters = tiles;
  }
  g.group_pairs = plan_group(g);
  g.a_policy = env_int("SDQ_TC2_APOLICY", 0);
  g.b_policy = env_int("SDQ_TC2_BPOLICY", 0);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(clusters * 2));
  cfg.blockDim = dim3(kNumThreads);
  const bool deep = tc2_config() == 61;
  cfg.dynamicSmemBytes = deep ? smem_bytes2(6, 1) : smem_bytes2(5, 2);
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see grid_dependency_wait()
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = env_int("SDQ_TC2_PDL", 1) ? 2 : 1;
  count_launch();
  cudaError_t e;
  // SDQ_TC2_PROBE=wideA: 4 x the A bytes per stage, 2 stages; =shallow: the same 2 stages with
  // the ordinary bytes (to separate the effect of the ring depth from that of the bytes)
  const char* probe = getenv("SDQ_TC2_PROBE");
  if (probe && !g.residual && probe[0] == 'w') {
    cfg.dynamicSmemBytes = smem_bytes2(2, 1, 4);
    e = cudaLaunchKernelEx(&cfg, qgemm_tc2_kernel<2, 1, false, 4>, ta, tb, outs, num_outs, ttail, g);
  } else if (probe && !g.residual && probe[0] == 's') {
    cfg.dynamicSmemBytes = smem_bytes2(2, 1, 1);
    e = cudaLaunchKernelEx(&cfg, qgemm_tc2_kernel<2, 1, false, 1>, ta, tb, outs, num_outs, ttail, g);
  } else if (g.residual) {
    e = deep ? cudaLaunchKernelEx(&cfg, qgemm_tc2_kernel<6, 1, true>, ta, tb, outs, num_outs, ttail, g)
             : cudaLaunchKernelEx(&cfg, qgemm_tc2_kernel<5, 2, true>, ta, tb, outs, num_outs, ttail, g);
  } else {
    e = deep ? cudaLaunchKernelEx(&cfg, qgemm_tc2_kernel<6, 1, false>, ta, tb, outs, num_outs, ttail, g)
             : cudaLaunchKernelEx(&cfg, qgemm_tc2_kernel<5, 2, false>, ta, tb, outs, num_outs, ttail, g);
  }
  if (e == cudaSuccess && tail > 0) {
    const int first_tail = (int)(tiles - tail);
    count_launch();  // (64 blocks per tile: 4, 16 and 256 measured 11, 4 and 1 us slower at 20 tiles)
    if (g.residual) tail_finalize_kernel<true><<<dim3((unsigned)tail, 64), 256, 0, s>>>(g, first_tail, g.group_pairs);
    else tail_finalize_kernel<false><<<dim3((unsigned)tail, 64), 256, 0, s>>>(g, first_tail, g.group_pairs);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace sdq
