// Exact-softmax attention on the Blackwell tensor cores: out[Lq,C] = softmax(q k^T / sqrt(hd)) v
// per head, the reference's blk::sdpa (src/model/blocks.h:60-66, src/model/blocks.cpp:113-199:
// fp32, no mask, scale 1/sqrt(head_dim)), for head_dim 128.
//
// Precision.  The reference is fp32 throughout and its outputs are compared at 1e-3 of the
// largest value, which a plain tf32 (10-bit mantissa) score cannot hold in the tails: an error of
// 2^-11 in q or k moves a score by ~1e-3 and exp() turns that into the same relative error of the
// weight.  So the scores are computed with three products per fp32 product (q = hi + lo,
// k = hi + lo with hi = tf32(x); hi*hi + lo*hi + hi*lo): the large term as tf32 MMAs, the two
// small cross terms (2^-11 of the product, so 8 mantissa bits are plenty) as bf16 MMAs, which
// take 16 instead of 8 elements of the head dimension per instruction.  The softmax weights and v are each split into two bf16
// numbers (16 mantissa bits together) and P*V is three bf16 MMAs (hi*hi + hi*lo + lo*hi): twice
// the rate of tf32 per MMA, the same shared-memory and tensor-memory footprint as one tf32 plane,
// and an error of ~1e-5 instead of the 3..6e-4 a single tf32 rounding of P and V leaves.  The row
// sums add the split weights, so numerator and denominator agree.
//
// Softmax without rescaling.  A first sweep over the keys finds each row's maximum from plain
// bf16 scores (any value near the true maximum serves as the offset, as long as numerator and
// denominator use the same one); a second sweep recomputes the scores accurately, exponentiates
// and accumulates P*V in tensor memory for the whole key range.  No accumulator is ever rescaled.
//
// One CTA per (128 query rows, head), persistent over these work items; 320 threads:
//   warp 10 lane 0: TMA producer of v^T (its own two-stage ring, released by the P*V MMAs, so
//                   the k ring -- released as soon as a block's scores are done -- runs ahead).
//   warp 0 lane 0 : TMA producer of k.  128 keys of bf16(k) per stage in sweep 1; per 64-key block
//                   k_hi, the bf16 planes of k and of v^T in sweep 2; 128-byte-swizzled boxes,
//                   two-stage ring.
//   warp 1 lane 0 : MMA issuer of the scores of the even key blocks.  S = Q K^T with Q as the
//   warp 12 lane 0: ... and of the odd key blocks.  A operand in TENSOR MEMORY, K from shared memory.
//   warp 11 lane 0: MMA issuer of O += P V, with P in tensor memory (written in place over S by
//                   the softmax warps) and V^T from shared memory.  Issuing a small MMA costs the
//                   issuing lane about as long as the tensor pipe needs for it, so the
//                   instruction streams come from three lanes.
//   warps 2..5    : softmax group A (one thread per query row): the first 32 keys of every block.
//   warps 6..9    : softmax group B: the other 32 keys.  Both groups finish the tile together:
//                   O / row sum -> staged boxes -> bulk tensor stores.
// Tensor memory (512 columns): Q_hi (tf32) 0..127, bf16(Q_lo) 128..191, bf16(Q_hi) 192..255,
// O 256..383, S/P buffers 384..447 and 448..511.  Every mbarrier wait is bounded like the GEMM kernels'.
#include "tc_common.cuh"
#include "tf32_split.cuh"

#include <cuda_bf16.h>

namespace sdq {
namespace {
using namespace tc;

constexpr int kHd = 128;            // head_dim this kernel is built for
constexpr int kBq = 128;            // query rows per work item
constexpr int kBkv = 64;            // keys per block
constexpr int kKTile = kBkv * kHd * 4;          // 32 KiB: one tf32 plane of a key block
constexpr int kVTile = kHd * kBkv * 4;          // 32 KiB: v^T of a key block
constexpr int kKStageBytes = 2 * kKTile;   // k_hi (tf32) + bf16(k_hi) + bf16(k_lo); sweep 1: 128 keys of k_hi
constexpr int kAStages = 2;                // per ring
constexpr int kAStageBytes = kKStageBytes + kVTile;  // both rings, one stage each
constexpr int kAThreads = kNumThreads + 96;  // + three warps: v^T producer, P*V issuer, second score issuer
constexpr int kABookBytes = 2304;    // row maxima and sums of both groups (2 KiB) + barriers
constexpr int kAAlignSlack = 768;    // to bring the dynamic base to a 1024-byte boundary
constexpr int kASmemBytes = kAStages * kAStageBytes + 8 * 4096 + kABookBytes + kAAlignSlack;  // 227 KiB
constexpr uint32_t kColQhi = 0, kColQloB = 128, kColQhiB = 192, kColO = 256, kColS = 384;
constexpr int kKbTile = kBkv * kHd * 2;         // 16 KiB: one bf16 plane of a key block
constexpr uint32_t kIdescS = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kBkv >> 3) << 17) |
                             ((uint32_t)(kBq >> 4) << 24);
// cross terms of the scores: kind::f16 with bf16 inputs (format 1), N = 64
constexpr uint32_t kIdescSb = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBkv >> 3) << 17) |
                              ((uint32_t)(kBq >> 4) << 24);
// P*V and the scores of sweep 1: kind::f16 with bf16 inputs (format 1), fp32 accumulator, N = 128
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kHd >> 3) << 17) |
                              ((uint32_t)(kBq >> 4) << 24);

// D[tmem] (+)= A[tmem] * B[smem]^T, tf32: the A operand (row i in lane i, K along the columns)
// is read from tensor memory.
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with bf16 operands (two K elements per 32-bit column of the A operand).
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t writes lane (base_lane + t).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

struct SdpaArgs {
  const float* q;   // [Lq, C]
  float* out;       // [Lq, C]
  int64_t Lq, Lk, C;
  int heads;
  float scale_log2e;  // (1 / sqrt(head_dim)) * log2(e)
  int* status;
};

__global__ void __launch_bounds__(kAThreads, 1)
    sdpa_tc_kernel(const __grid_constant__ CUtensorMap tmap_k_hib128,
                   const __grid_constant__ CUtensorMap tmap_k_hi,
                   const __grid_constant__ CUtensorMap tmap_k_hib,
                   const __grid_constant__ CUtensorMap tmap_k_lob,
                   const __grid_constant__ CUtensorMap tmap_vt_hi,
                   const __grid_constant__ CUtensorMap tmap_vt_lo,
                   const __grid_constant__ CUtensorMap tmap_out, SdpaArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_staging = base + kAStages * kAStageBytes;
  uint8_t* book = smem + kAStages * kAStageBytes + 8 * 4096;
  // row maxima and row sums of the two softmax groups, then the barriers
  float* x_max = reinterpret_cast<float*>(book);          // [2][128]
  float* x_sum = reinterpret_cast<float*>(book + 1024);   // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(book + 2048);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_full = bar0;               // [2]  k ring: TMA bytes landed
  const uint32_t bar_empty = bar0 + 16;         // [2]  k ring: stage read by its last MMA
  const uint32_t bar_sfull = bar0 + 32;         // [2]  scores of a block complete
  const uint32_t bar_s1free = bar0 + 48;        // [2]  sweep 1: scores read by the softmax group
  const uint32_t bar_pready = bar0 + 64;        // [2]  sweep 2: weights written over the scores
  const uint32_t bar_pvdone = bar0 + 80;        // [2]  sweep 2: P*V of a block complete
  const uint32_t bar_qready = bar0 + 96;        // Q planes in tensor memory
  const uint32_t bar_mready = bar0 + 104;       // both groups published their row maxima
  const uint32_t bar_lready = bar0 + 112;       // both groups published their row sums
  const uint32_t bar_ofull = bar0 + 120;        // every MMA of the work item complete
  const uint32_t bar_ofree = bar0 + 128;        // O read out: the next item may overwrite it
  const uint32_t bar_vfull = bar0 + 136;        // [2]  v^T ring
  const uint32_t bar_vempty = bar0 + 152;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (base - raw > (uint32_t)kAAlignSlack) {
    // the dynamic shared memory starts further from a 1024-byte boundary than the launch
    // budgeted for: report it instead of running past the allocation
    if (threadIdx.x == 0) atomicCAS(g.status, 0, 0xb00 | 1);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = (int)((g.Lq + kBq - 1) / kBq);
  const int nblk = (int)((g.Lk + kBkv - 1) / kBkv);
  const int nblk1 = (int)((g.Lk + 2 * kBkv - 1) / (2 * kBkv));  // sweep 1 walks 128 keys at a time
  const int num_items = nqt * g.heads;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; i++) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_s1free + 8 * i, 8);
      mbar_init(bar_pready + 8 * i, 8);
      mbar_init(bar_pvdone + 8 * i, 1);
      mbar_init(bar_vfull + 8 * i, 1);
      mbar_init(bar_vempty + 8 * i, 1);
    }
    mbar_init(bar_qready, 4);
    mbar_init(bar_mready, 8);
    mbar_init(bar_lready, 8);
    mbar_init(bar_ofull, 1);
    mbar_init(bar_ofree, 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tmap_k_hib128);
    prefetch_tmap(&tmap_k_hi);
    prefetch_tmap(&tmap_k_hib);
    prefetch_tmap(&tmap_k_lob);
    prefetch_tmap(&tmap_vt_hi);
    prefetch_tmap(&tmap_vt_lo);
    prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer of k
      const uint64_t keep = policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int h = item / nqt;
        // sweep 1: bf16(k_hi) only, 128 keys per stage (two boxes of 128 keys x 64 dims)
        for (int j = 0; j < nblk1; j++) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x800 | 1);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t st = base + stage * kKStageBytes;
          mbar_expect_tx(full, 2 * kKbTile);
          for (int i = 0; i < 2; i++)
            tma_load_2d_hint(st + i * 16384, &tmap_k_hib128, full, h * kHd + 64 * i, j * 2 * kBkv, keep);
          if (++stage == kAStages) { stage = 0; phase ^= 1u; }
        }
        // sweep 2: k_hi (boxes of 64 keys x 32 dims), bf16(k_hi) and bf16(k_lo) (boxes of 64 keys
        // x 64 dims)
        for (int j = 0; ok && j < nblk; j++) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x800 | 2);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t st = base + stage * kKStageBytes;
          mbar_expect_tx(full, kKStageBytes);
          for (int i = 0; i < 4; i++)
            tma_load_2d_hint(st + i * 8192, &tmap_k_hi, full, h * kHd + 32 * i, j * kBkv, keep);
          for (int i = 0; i < 2; i++) {
            tma_load_2d_hint(st + kKTile + i * 8192, &tmap_k_hib, full, h * kHd + 64 * i, j * kBkv, keep);
            tma_load_2d_hint(st + kKTile + kKbTile + i * 8192, &tmap_k_lob, full, h * kHd + 64 * i, j * kBkv, keep);
          }
          if (++stage == kAStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 10) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer of v^T (sweep 2 only):
      // the two bf16 planes, one box of 128 dims x 64 keys each
      const uint64_t keep = policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int h = item / nqt;
        for (int j = 0; j < nblk; j++) {
          ok = mbar_wait(bar_vempty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x800 | 3);
          if (!ok) break;
          const uint32_t full = bar_vfull + 8 * stage;
          const uint32_t st = base + kAStages * kKStageBytes + stage * kVTile;
          mbar_expect_tx(full, kVTile);
          tma_load_2d_hint(st, &tmap_vt_hi, full, j * kBkv, h * kHd, keep);
          tma_load_2d_hint(st + 16384, &tmap_vt_lo, full, j * kBkv, h * kHd, keep);
          if (++stage == kAStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == 12) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuers of the scores: this lane
      // takes the blocks of one parity (warp 1 the even ones, warp 12 the odd ones) in both
      // sweeps, i.e. always the same score buffer.  The k ring is shared: block number `seq` of
      // the CTA's whole run sits in stage seq & 1, whose full barrier completes its phase
      // (seq >> 1) & 1 for it.
      const uint32_t par = warp == 1 ? 0u : 1u;
      uint32_t sfree_ph = 0;                    // completed phases of s1free[par]
      uint32_t pv_ph = 0;                       // completed phases of pvdone[par]
      uint32_t q_ph = 0, m_ph = 0, ofree_ph = 0;
      uint32_t seq0 = 0;                        // k-ring sequence number of the item's first block
      bool ok = true;
      // scores of a block from the operands in `st`: the two small cross terms first (bf16, 16
      // dims per instruction), then the large term (tf32, 8 dims per instruction)
      auto issue_scores = [&](uint32_t st) {
        const uint32_t d = tmem_base + kColS + par * kBkv;
#pragma unroll
        for (int ks = 0; ks < kHd / 16; ks++) {
          const uint32_t off = (uint32_t)((ks >> 2) * 8192);
          const uint64_t adv = (uint64_t)((ks & 3) * 2);
          const uint64_t k_hib = make_smem_desc(st + kKTile + off) + adv;
          const uint64_t k_lob = make_smem_desc(st + kKTile + kKbTile + off) + adv;
          umma_bf16_ts(d, tmem_base + kColQloB + ks * 8, k_hib, kIdescSb, (uint32_t)(ks != 0));
          umma_bf16_ts(d, tmem_base + kColQhiB + ks * 8, k_lob, kIdescSb, 1u);
        }
#pragma unroll
        for (int ks = 0; ks < kHd / 8; ks++) {
          const uint64_t k_hi = make_smem_desc(st + (uint32_t)((ks >> 2) * 8192)) + (uint64_t)((ks & 3) * 2);
          umma_tf32_ts(d, tmem_base + kColQhi + ks * 8, k_hi, kIdescS, 1u);
        }
      };
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        ok = mbar_wait_spin(bar_qready, q_ph, abort_flag, g.status, 0x900 | 1);
        q_ph ^= 1u;
        if (!ok) break;
        // the previous item's O has been read out: sweep 1 borrows its columns
        ok = mbar_wait_spin(bar_ofree, ofree_ph ^ 1u, abort_flag, g.status, 0x900 | 5);
        ofree_ph ^= 1u;
        if (!ok) break;
        tc_fence_after();
        // ---- sweep 1: bf16 scores for the row maxima (8 mantissa bits are ample for an offset),
        // 128 keys and 16 dims per MMA; the even blocks go to the score columns (384..511), the
        // odd ones to the idle O columns (256..383)
        for (int j = (int)par; j < nblk1; j += 2) {
          const uint32_t seq = seq0 + (uint32_t)j, stage = seq & 1u;
          ok = mbar_wait_spin(bar_full + 8 * stage, (seq >> 1) & 1u, abort_flag, g.status, 0x900 | 2);
          if (!ok) break;
          ok = mbar_wait_spin(bar_s1free + 8 * par, sfree_ph ^ 1u, abort_flag, g.status, 0x900 | 3);
          if (!ok) break;
          sfree_ph ^= 1u;
          tc_fence_after();
          const uint32_t st = base + stage * kKStageBytes;
          const uint32_t d = tmem_base + (par ? kColO : kColS);
#pragma unroll
          for (int ks = 0; ks < kHd / 16; ks++) {
            const uint64_t kd = make_smem_desc(st + (uint32_t)((ks >> 2) * 16384)) + (uint64_t)((ks & 3) * 2);
            umma_bf16_ts(d, tmem_base + kColQhiB + ks * 8, kd, kIdescPV, (uint32_t)(ks != 0));
          }
          umma_commit(bar_empty + 8 * stage);
          umma_commit(bar_sfull + 8 * par);
        }
        if (!ok) break;
        // the softmax groups have read every score of sweep 1 and published the maxima
        ok = mbar_wait_spin(bar_mready, m_ph, abort_flag, g.status, 0x900 | 4);
        m_ph ^= 1u;
        if (!ok) break;
        tc_fence_after();
        // ---- sweep 2: accurate scores of this lane's blocks.  The buffer is free again when the
        // P*V of the block two back has consumed its weights; a k stage is released as soon as
        // the scores that read it are done.
        bool any = false;
        for (int j = (int)par; j < nblk; j += 2) {
          const uint32_t seq = seq0 + (uint32_t)(nblk1 + j), stage = seq & 1u;
          ok = mbar_wait_spin(bar_full + 8 * stage, (seq >> 1) & 1u, abort_flag, g.status, 0x900 | 7);
          if (!ok) break;
          if (any) {
            ok = mbar_wait_spin(bar_pvdone + 8 * par, pv_ph, abort_flag, g.status, 0x900 | 8);
            if (!ok) break;
            pv_ph ^= 1u;
          }
          tc_fence_after();
          issue_scores(base + stage * kKStageBytes);
          umma_commit(bar_empty + 8 * stage);
          umma_commit(bar_sfull + 8 * par);
          any = true;
        }
        if (!ok) break;
        if (any) {  // the completion of this lane's last block, so that the parity stays in step
          ok = mbar_wait_spin(bar_pvdone + 8 * par, pv_ph, abort_flag, g.status, 0x900 | 10);
          pv_ph ^= 1u;
          if (!ok) break;
        }
        seq0 += (uint32_t)(nblk1 + nblk);
      }
    }
  } else if (warp == 11) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuer of P*V
      uint32_t vstage = 0, vphase = 0;
      uint32_t pready_ph[2] = {0, 0};
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        // (O is free: every softmax warp released the previous item's O before it could arrive
        // on this item's first pready)
        for (int j = 0; j < nblk; j++) {
          const uint32_t buf = (uint32_t)(j & 1);
          ok = mbar_wait_spin(bar_pready + 8 * buf, pready_ph[buf], abort_flag, g.status, 0x900 | 9);
          if (!ok) break;
          pready_ph[buf] ^= 1u;
          ok = mbar_wait_spin(bar_vfull + 8 * vstage, vphase, abort_flag, g.status, 0x900 | 11);
          if (!ok) break;
          tc_fence_after();
          const uint32_t vt = base + kAStages * kKStageBytes + vstage * kVTile;
          const uint32_t pcol = tmem_base + kColS + buf * kBkv;
#pragma unroll
          for (int ks = 0; ks < kBkv / 16; ks++) {
            // 16 keys per kind::f16 instruction = 32 bytes of a v^T row: +2 in the address field.
            // The weights of keys 16ks.. sit in 8 columns: hi at (ks>>1)*32 + (ks&1)*8, lo 16 further.
            const uint64_t v_hi = make_smem_desc(vt) + (uint64_t)(ks * 2);
            const uint64_t v_lo = make_smem_desc(vt + 16384) + (uint64_t)(ks * 2);
            const uint32_t p_hi = pcol + (uint32_t)((ks >> 1) * 32 + (ks & 1) * 8);
            umma_bf16_ts(tmem_base + kColO, p_hi + 16, v_hi, kIdescPV, (uint32_t)((j | ks) != 0));
            umma_bf16_ts(tmem_base + kColO, p_hi, v_lo, kIdescPV, 1u);
            umma_bf16_ts(tmem_base + kColO, p_hi, v_hi, kIdescPV, 1u);
          }
          umma_commit(bar_vempty + 8 * vstage);
          umma_commit(bar_pvdone + 8 * buf);
          if (++vstage == kAStages) { vstage = 0; vphase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(bar_ofull);  // every P*V of the item (and so every MMA before them) is complete
      }
    }
  } else {
    // -------------------------------------------------- softmax groups + epilogue (8 warps)
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;        // 0: keys 0..31 of every block, 1: keys 32..63
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t box = smem_staging + (uint32_t)((warp - 2) * 4096);
    const uint64_t stream_policy = policy_evict_first();
    const uint32_t s_col = tmem_base + kColS + (uint32_t)grp * 32 + lane_base;  // + buffer * kBkv
    uint32_t sfull_ph[2] = {0, 0};
    uint32_t m_ph = 0, l_ph = 0, ofull_ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      const int h = item / nqt, qt = item - h * nqt;
      const int64_t q0 = (int64_t)qt * kBq;
      const int64_t row = q0 + row_in_tile;
      if (grp == 0) {
        // this thread's query row -> tensor memory (zeros past Lq): the tf32 plane q_hi, and
        // bf16(q - q_hi) and bf16(q_hi) for the cross terms, two elements per column
        const float* qrow = g.q + row * g.C + (int64_t)h * kHd;
#pragma unroll 1
        for (int c = 0; c < kHd / 64; c++) {
          uint32_t lob[32], hib[32];
#pragma unroll 1
          for (int half_c = 0; half_c < 2; half_c++) {
            uint32_t hi[32];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
              if (row < g.Lq) v = *reinterpret_cast<const float4*>(qrow + c * 64 + half_c * 32 + j);
              const float xs[4] = {v.x, v.y, v.z, v.w};
              float a[4], b[4];
#pragma unroll
              for (int t = 0; t < 4; t++) {
                split_tf32(xs[t], a[t], b[t]);
                hi[j + t] = __float_as_uint(a[t]);
              }
#pragma unroll
              for (int t = 0; t < 4; t += 2) {
                const __nv_bfloat162 pl = __floats2bfloat162_rn(b[t], b[t + 1]);  // lower dim in the low half
                const __nv_bfloat162 ph = __floats2bfloat162_rn(a[t], a[t + 1]);
                lob[half_c * 16 + ((j + t) >> 1)] = *reinterpret_cast<const uint32_t*>(&pl);
                hib[half_c * 16 + ((j + t) >> 1)] = *reinterpret_cast<const uint32_t*>(&ph);
              }
            }
            tmem_st_32x32(tmem_base + kColQhi + c * 64 + half_c * 32 + lane_base, hi);
          }
          tmem_st_32x32(tmem_base + kColQloB + c * 32 + lane_base, lob);
          tmem_st_32x32(tmem_base + kColQhiB + c * 32 + lane_base, hib);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_qready);
      }
      // ---- sweep 1: the row maximum over this group's blocks (raw dot products)
      float m = -INFINITY;
      for (int j = 0; j < nblk1; j++) {
        const uint32_t buf = (uint32_t)(j & 1);
        ok = mbar_wait_warp(bar_sfull + 8 * buf, sfull_ph[buf], abort_flag, g.status, 0xa00 | 1);
        sfull_ph[buf] ^= 1u;
        if (!ok) break;
        tc_fence_after();
        // this group's 64 of the block's 128 keys
        const uint32_t x_col = tmem_base + (buf ? kColO : kColS) + (uint32_t)grp * 64 + lane_base;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(x_col, r0);
        tmem_ld_32x32(x_col + 32, r1);
        tmem_ld_wait();
        const int64_t key0 = (int64_t)j * 2 * kBkv + grp * 64;
#pragma unroll
        for (int t = 0; t < 32; t++) {
          if (key0 + t < g.Lk) m = fmaxf(m, __uint_as_float(r0[t]));
          if (key0 + 32 + t < g.Lk) m = fmaxf(m, __uint_as_float(r1[t]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s1free + 8 * buf);
      }
      if (!ok) break;
      x_max[grp * kBq + row_in_tile] = m;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_mready);
      ok = mbar_wait_warp(bar_mready, m_ph, abort_flag, g.status, 0xa00 | 2);
      m_ph ^= 1u;
      if (!ok) break;
      m = fmaxf(x_max[row_in_tile], x_max[kBq + row_in_tile]);
      // ---- sweep 2: weights p = exp((s - m) * scale), rounded to tf32, written over the scores
      float l = 0.0f;
      for (int j = 0; j < nblk; j++) {
        const uint32_t buf = (uint32_t)(j & 1);
        ok = mbar_wait_warp(bar_sfull + 8 * buf, sfull_ph[buf], abort_flag, g.status, 0xa00 | 3);
        sfull_ph[buf] ^= 1u;
        if (!ok) break;
        tc_fence_after();
        {
          uint32_t r[32];
          tmem_ld_32x32(s_col + buf * kBkv, r);
          tmem_ld_wait();
          const int64_t key0 = (int64_t)j * kBkv + grp * 32;
          const int valid = (int)min((int64_t)32, g.Lk - key0);  // < 32 only in the last block
          // this group's 32 columns become: 16 columns of bf16 pairs p_hi, then 16 of p_lo.
          // Two weights at a time: one cvt packs the pair of high parts, whose fp32 values are
          // the two halves of that word shifted up; the low parts are what is left, packed by a
          // second cvt.  The row sum adds the weights themselves (they differ from hi + lo by
          // 2^-17 at most).
          uint32_t w[32];
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            float p0 = 0.0f, p1 = 0.0f;
            const float e0 = __fmul_rn(__fsub_rn(__uint_as_float(r[t]), m), g.scale_log2e);
            const float e1 = __fmul_rn(__fsub_rn(__uint_as_float(r[t + 1]), m), g.scale_log2e);
            asm("ex2.approx.f32 %0, %1;" : "=f"(p0) : "f"(e0));
            asm("ex2.approx.f32 %0, %1;" : "=f"(p1) : "f"(e1));
            if (t >= valid) p0 = 0.0f;
            if (t + 1 >= valid) p1 = 0.0f;
            l += __fadd_rn(p0, p1);
            uint32_t hi2, lo2;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi2) : "f"(p1), "f"(p0));  // first source -> upper half
            const float h0 = __uint_as_float(hi2 << 16), h1 = __uint_as_float(hi2 & 0xffff0000u);
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo2) : "f"(__fsub_rn(p1, h1)), "f"(__fsub_rn(p0, h0)));
            w[t >> 1] = hi2;
            w[16 + (t >> 1)] = lo2;
          }
          tmem_st_32x32(s_col + buf * kBkv, w);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pready + 8 * buf);
      }
      if (!ok) break;
      x_sum[grp * kBq + row_in_tile] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_lready);
      ok = mbar_wait_warp(bar_lready, l_ph, abort_flag, g.status, 0xa00 | 4);
      l_ph ^= 1u;
      if (!ok) break;
      l = x_sum[row_in_tile] + x_sum[kBq + row_in_tile];
      const float inv = __fdiv_rn(1.0f, l);
      // ---- epilogue: O / l, this group's two 32-column chunks
      ok = mbar_wait_warp(bar_ofull, ofull_ph, abort_flag, g.status, 0xa00 | 5);
      ofull_ph ^= 1u;
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 2 * grp; c < 2 * grp + 2; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + kColO + c * 32 + lane_base, r);
        tmem_ld_wait();
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st_shared_v4(box + (uint32_t)(lane * 128 + (((j >> 2) ^ (lane & 7)) << 4)),
                       make_float4(__fmul_rn(__uint_as_float(r[j]), inv), __fmul_rn(__uint_as_float(r[j + 1]), inv),
                                   __fmul_rn(__uint_as_float(r[j + 2]), inv), __fmul_rn(__uint_as_float(r[j + 3]), inv)));
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d_hint(&tmap_out, box, h * kHd + c * 32, (int)(q0 + quarter * 32), stream_policy);
          bulk_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ofree);
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
    tmem_dealloc(tmem_base, 512);
  }
}

// k -> the tf32 plane k_hi and, for the cross terms, bf16(k_hi) and bf16(k - k_hi).
__global__ void __launch_bounds__(256) split_planes_kernel(const float* __restrict__ x, int64_t n,
                                                           float* __restrict__ hi,
                                                           __nv_bfloat16* __restrict__ hib,
                                                           __nv_bfloat16* __restrict__ lob) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    float a, b;
    split_tf32(x[i], a, b);
    hi[i] = a;
    hib[i] = __float2bfloat16_rn(a);
    lob[i] = __float2bfloat16_rn(b);
  }
}

// v [Lk, C] -> two bf16 planes of v^T, each [C, ld] (ld >= Lk, a multiple of 8; the padding is
// zero): hi = bf16(v), lo = bf16(v - hi).
__global__ void __launch_bounds__(256) transpose_split_bf16_kernel(const float* __restrict__ v, int64_t Lk,
                                                                   int64_t C, int64_t ld,
                                                                   __nv_bfloat16* __restrict__ vt_hi,
                                                                   __nv_bfloat16* __restrict__ vt_lo) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t k0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
  for (int r = ty; r < 32; r += 8)
    tile[r][tx] = (k0 + r < Lk && c0 + tx < C) ? v[(k0 + r) * C + c0 + tx] : 0.0f;
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    if (c0 + r < C && k0 + tx < ld) {
      const float x = tile[tx][r];
      const __nv_bfloat16 h = __float2bfloat16_rn(x);
      const float rest = isfinite(x) ? __fsub_rn(x, __bfloat162float(h)) : 0.0f;
      vt_hi[(c0 + r) * ld + k0 + tx] = h;
      vt_lo[(c0 + r) * ld + k0 + tx] = __float2bfloat16_rn(rest);
    }
  }
}

// Any head_dim / alignment: one warp per (query row, head), exact fp32 on the CUDA cores, three
// passes over the keys (maximum, sum, weighted values).
__global__ void __launch_bounds__(256) sdpa_simt_kernel(const float* __restrict__ q,
                                                        const float* __restrict__ k,
                                                        const float* __restrict__ v, int64_t Lq,
                                                        int64_t Lk, int64_t C, int heads,
                                                        float scale, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t hd = C / heads;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t it = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); it < Lq * heads; it += warps) {
    const int64_t i = it / heads, h = it - i * heads;
    const float* qi = q + i * C + h * hd;
    auto score = [&](int64_t t) {
      const float* kt = k + t * C + h * hd;
      float d = 0.0f;
      for (int64_t c = lane; c < hd; c += 32) d = fmaf(qi[c], kt[c], d);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      return d * scale;
    };
    float mx = -INFINITY;
    for (int64_t t = 0; t < Lk; t++) mx = fmaxf(mx, score(t));
    float sum = 0.0f;
    for (int64_t t = 0; t < Lk; t++) sum += expf(score(t) - mx);
    const float inv = 1.0f / sum;
    for (int64_t c0 = 0; c0 < hd; c0 += 32) {
      float o = 0.0f;
      for (int64_t t = 0; t < Lk; t++) {
        const float w = expf(score(t) - mx) * inv;
        if (c0 + lane < hd) o = fmaf(w, v[t * C + h * hd + c0 + lane], o);
      }
      if (c0 + lane < hd) out[i * C + h * hd + c0 + lane] = o;
    }
  }
}

// v^T plane [C, ld] bf16, box = 128 rows x 64 keys (128 bytes), 128-byte swizzle.
bool make_tmap_vt(CUtensorMap* map, const void* ptr, int64_t C, int64_t Lk, int64_t ld, std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)Lk, (cuuint64_t)C};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBkv, (cuuint32_t)kHd};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(v^T) failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

// bf16 plane of k [Lk, C], box = box_keys keys x 64 dims (128 bytes), 128-byte swizzle.
bool make_tmap_kb(CUtensorMap* map, const void* ptr, int64_t Lk, int64_t C, int box_keys, std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)Lk};
  cuuint64_t strides[1] = {(cuuint64_t)C * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_keys};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(bf16 k plane) failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

bool make_tmap_2d_f32(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t pitch_elems,
                      int box_rows, std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(attention operand) failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

}  // namespace

int sdpa_setup(std::string* why) {
  cudaError_t e = cudaFuncSetAttribute(sdpa_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kASmemBytes);
  if (e != cudaSuccess) {
    if (why) *why = std::string("cudaFuncSetAttribute(attention, max dynamic smem): ") + cudaGetErrorString(e);
    return SDQ_ERR_CUDA;
  }
  return SDQ_OK;
}

size_t sdpa_scratch_bytes(int64_t Lk, int64_t C) {
  const int64_t ld = (Lk + 7) / 8 * 8;
  return (size_t)(Lk * C) * 4 + (size_t)(2 * Lk * C + 2 * C * ld) * 2;  // k_hi fp32; k and v^T hi, lo bf16
}

cudaError_t launch_sdpa(const float* q, const float* k, const float* v, int64_t Lq, int64_t Lk,
                        int64_t C, int heads, float* out, float* scratch, int* status,
                        uint32_t flags, int sm_count, cudaStream_t s, std::string* why) {
  if (Lq <= 0 || C <= 0 || heads <= 0) return cudaSuccess;
  if (Lk <= 0) return cudaMemsetAsync(out, 0, (size_t)Lq * C * 4, s);  // no keys: the sums are empty
  const int64_t hd = C / heads;
  const float scale = 1.0f / sqrtf((float)hd);
  const bool tc_ok = g_encode != nullptr && !(flags & SDQ_FORCE_SIMT) && hd == kHd && C == (int64_t)heads * kHd &&
                     ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(scratch)) & 15) == 0 &&
                     Lq < (int64_t(1) << 31) && Lk < (int64_t(1) << 31);
  if (!tc_ok) {
    int64_t blocks = (Lq * heads + 7) / 8;
    if (blocks > (int64_t)sm_count * 8) blocks = (int64_t)sm_count * 8;
    count_launch();
    sdpa_simt_kernel<<<(unsigned)blocks, 256, 0, s>>>(q, k, v, Lq, Lk, C, heads, scale, out);
    return cudaGetLastError();
  }
  const int64_t ld = (Lk + 7) / 8 * 8;
  float* k_hi = scratch;
  __nv_bfloat16* k_hib = reinterpret_cast<__nv_bfloat16*>(scratch + Lk * C);
  __nv_bfloat16* k_lob = k_hib + Lk * C;
  __nv_bfloat16* vt_hi = k_lob + Lk * C;
  __nv_bfloat16* vt_lo = vt_hi + C * ld;
  int64_t blocks = (Lk * C + 255) / 256;
  if (blocks > (int64_t)sm_count * 16) blocks = (int64_t)sm_count * 16;
  count_launch(2);
  split_planes_kernel<<<(unsigned)blocks, 256, 0, s>>>(k, Lk * C, k_hi, k_hib, k_lob);
  dim3 tgrid((unsigned)((C + 31) / 32), (unsigned)((ld + 31) / 32));
  transpose_split_bf16_kernel<<<tgrid, 256, 0, s>>>(v, Lk, C, ld, vt_hi, vt_lo);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  CUtensorMap t_khi128, t_khi, t_khib, t_klob, t_vt_hi, t_vt_lo, t_out;
  if (!make_tmap_kb(&t_khi128, k_hib, Lk, C, 2 * kBkv, why) ||
      !make_tmap_2d_f32(&t_khi, k_hi, Lk, C, C, kBkv, why) || !make_tmap_kb(&t_khib, k_hib, Lk, C, kBkv, why) ||
      !make_tmap_kb(&t_klob, k_lob, Lk, C, kBkv, why) ||
      !make_tmap_vt(&t_vt_hi, vt_hi, C, Lk, ld, why) || !make_tmap_vt(&t_vt_lo, vt_lo, C, Lk, ld, why) ||
      !make_out_tmap(&t_out, out, Lq, C, why))
    return cudaErrorInvalidValue;
  SdpaArgs g;
  g.q = q; g.out = out; g.Lq = Lq; g.Lk = Lk; g.C = C; g.heads = heads;
  g.scale_log2e = scale * 1.4426950408889634f;
  g.status = status;
  const int64_t items = ((Lq + kBq - 1) / kBq) * heads;
  count_launch();
  sdpa_tc_kernel<<<(unsigned)(items < sm_count ? items : sm_count), kAThreads, kASmemBytes, s>>>(
      t_khi128, t_khi, t_khib, t_klob, t_vt_hi, t_vt_lo, t_out, g);
  return cudaGetLastError();
}

}  // namespace sdq
