// Exact-softmax attention on the Blackwell tensor cores: out[Lq,C] = softmax(q k^T / sqrt(hd)) v
// per head, the reference's blk::sdpa (src/model/blocks.h:60-66, src/model/blocks.cpp:113-199:
// fp32, no mask, scale 1/sqrt(head_dim)), for head_dim 128.
//
// Precision.  The reference is fp32 throughout and its outputs are compared at 1e-3 of the
// largest value, which a single 11-bit rounding of q and k cannot hold in the tails: an error of
// 2^-11 in q or k moves a score by ~1e-3 and exp() turns that into the same relative error of the
// weight.  So every operand is split into two fp16 numbers, x * 2^sh = hi + lo with hi = fp16(.)
// and lo = fp16(. - hi) (22 mantissa bits together), and every product is three fp16 MMAs
// (hi*hi + lo*hi + hi*lo, fp32 accumulation), for the scores and for P*V alike.  fp16 carries the
// same 11 bits as tf32 but takes 16 instead of 8 elements of the contraction per instruction and
// half the shared and tensor memory, which is what lets a key block be 128 keys wide.  The
// powers of two 2^sh bring each operand's largest magnitude to [2^14, 2^15), so nothing overflows
// and elements down to 2^-29 of the largest keep all their bits: one shift per query row (found by
// the thread that owns the row), one for the whole of k and one for v (an absmax pass before the
// split), a constant 2^10 for the softmax weights.  They are undone exactly: the row's and k's in
// the factor the scores are multiplied by anyway, v's in the final 1 / row sum; the weights' cancels.
// The row sums add the weights themselves, so numerator and denominator agree.
//
// One sweep over the keys.  Each row carries a running offset m (a raw dot product): weights are
// p = 2^10 exp((s - m) scale), O accumulates P*V in tensor memory for the whole key range.  Any
// value near the row's maximum serves as the offset, as long as numerator and denominator use
// the same one, and the fp16 weights have room up to 2^15.8: so the offset only moves when a
// block's maximum exceeds it by more than 4 log2 units, and only then O and the row sum are
// scaled down (by the softmax threads, after the P*V that was accumulating into O has
// completed) -- on ordinary data in the first block or two of a row, never afterwards.  The two
// threads that share a row (one per 64 of a block's 128 keys) exchange their block maxima
// through shared memory, so both always hold the same offset.  A row whose scores can be so
// large (head_dim * max|q_row| * max|k| / sqrt(head_dim) above 2^19 log2 units) that the dropped
// lo*lo terms, 2^-22 of the products, would reach the weights is marked and recomputed
// afterwards in plain fp32 on the CUDA cores by the kernel that also serves the other head
// sizes; so is a row whose sum is not finite or whose weights left fp16's range.
//
// One CTA per (128 query rows, head), persistent over these work items; 416 threads:
//   warp 0 lane 0 : TMA producer of k: a ring of four 32 KiB slots, one plane of 128 keys each
//                   (128-byte-swizzled boxes of 128 keys x 64 dims), hi then lo per key block;
//                   released as soon as a block's scores are done (a load takes ~1500 cycles
//                   from release to landed).
//   warp 10 lane 0: TMA producer of v^T (hi and lo planes, 64 keys per stage, its own three-stage
//                   ring released by the P*V MMAs).
//   warp 1 lane 0 : MMA issuer of the scores of the even key blocks.  S = Q K^T with Q as the
//   warp 12 lane 0: ... and of the odd key blocks.  A operand in TENSOR MEMORY, K from shared memory.
//   warp 11 lane 0: MMA issuer of O += P V, with P in tensor memory (written in place over S by
//                   the softmax warps) and V^T from shared memory.  A lane gets one of these
//                   MMAs out every ~90-125 cycles whatever its width, the tensor pipe needs 64
//                   for a 128-wide one: the pipe is full when two lanes issue at the same time.
//   warps 2..5    : softmax group A (one thread per query row): the first 64 keys of every block.
//   warps 6..9    : softmax group B: the other 64 keys.  Both groups finish the tile together:
//                   O / row sum, each thread storing its row's 128-byte pieces.
// Tensor memory (512 columns, two fp16 per column for the A operands): Q_hi 0..63, Q_lo 64..127,
// O 128..255, S/P buffers 256..383 and 384..511.  Every mbarrier wait is bounded like the GEMM
// kernels'.
#include "tc_common.cuh"

#include <cuda_fp16.h>

namespace sdq {
namespace {
using namespace tc;

constexpr int kHd = 128;            // head_dim this kernel is built for
constexpr int kBq = 128;            // query rows per work item
constexpr int kBkv = 128;           // keys per block
constexpr int kVKeys = 64;          // keys per stage of the v^T ring
constexpr int kKPlane = kBkv * kHd * 2;         // 32 KiB: one fp16 plane of a key block
constexpr int kVPlane = kHd * kVKeys * 2;       // 16 KiB: one fp16 plane of 64 keys of v^T
constexpr int kVStageBytes = 2 * kVPlane;       // v^T hi + lo
constexpr int kKSlots = 4;                 // k ring: slots of one plane (a key block takes two: hi, lo)
constexpr int kVStages = 3;                // v^T ring
constexpr int kARingBytes = kKSlots * kKPlane + kVStages * kVStageBytes;   // 224 KiB
constexpr int kAThreads = kNumThreads + 96;  // + three warps: v^T producer, P*V issuer, second score issuer
constexpr int kABookBytes = 2304;    // row maxima and sums of both groups (2 KiB) + barriers
constexpr int kAAlignSlack = 768;    // to bring the dynamic base to a 1024-byte boundary
constexpr int kASmemBytes = kARingBytes + kABookBytes + kAAlignSlack;  // 227 KiB
constexpr uint32_t kColQhi = 0, kColQlo = 64, kColO = 128, kColS = 256;
constexpr float kPShift = 10.0f;     // the softmax weights are carried as p * 2^10 (p relative to the
                                     // row's running offset: at most 2^kRescaleStep)
constexpr uint32_t kPHalfTop = 0x7b00;  // fp16 bits of 2^15.8: no finite weight gets there
constexpr float kRowSumFloor = 8.0f;    // (a row sum is at least 2^10 / 2^kRescaleStep unless something is not finite)
constexpr float kRescaleStep = 4.0f;    // log2 units by which a block's maximum may exceed the running
                                        // offset before the offset moves (weights stay below 2^14)
constexpr float kScoreBound = 524288.0f;  // 2^19 log2 units: above this bound on sum |q_d k_d| the
                                          // dropped lo*lo terms (2^-22 of it) would show in the weights
constexpr int kOperandTop = 14;      // operands are scaled so that their largest magnitude is in [2^14, 2^15)
// kind::f16 with fp16 inputs (format 0), fp32 accumulator, M = 128, N = 128: the scores (N = keys)
// and P*V (N = head dims)
constexpr uint32_t kIdescH = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(128 >> 3) << 17) |
                             ((uint32_t)(kBq >> 4) << 24);

// The power of two that brings a magnitude with these fp32 bits to [2^14, 2^15), as an exponent;
// 0 for zero, subnormal, infinite or NaN magnitudes, and limited so that 2^sh is a normal float.
__host__ __device__ __forceinline__ int operand_shift(uint32_t absbits) {
  const int e = (int)(absbits >> 23) & 0xff;
  if (e == 0 || e == 255) return 0;
  const int sh = kOperandTop - (e - 127);
  return sh < -100 ? -100 : (sh > 100 ? 100 : sh);
}
__device__ __forceinline__ float pow2f(int sh) {  // |sh| <= 126
  return __uint_as_float((uint32_t)(127 + sh) << 23);
}
// x -> the fp16 pair (hi, lo) of two scaled values, lower index in the low half
__device__ __forceinline__ void split_f16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  const __half2 h = __floats2half2_rn(x0, x1);
  const float2 f = __half22float2(h);
  const __half2 l = __floats2half2_rn(__fsub_rn(x0, f.x), __fsub_rn(x1, f.y));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// D[tmem] (+)= A[tmem] * B[smem]^T, kind::f16: the A operand (row i in lane i, two K elements per
// 32-bit column, the lower index in the low half) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
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
  const uint32_t* absmax;  // fp32 bits of max |k| and max |v|
  uint8_t* redo;           // [Lq, heads], zero on entry: 1 = recompute this row in plain fp32
  int64_t Lq, Lk, C;
  int heads;
  int v_lo;          // 1: P*V uses both planes of v^T (three MMAs per product), 0: the hi plane only (two)
  int k_lo;          // 1: the scores use both planes of k (three MMAs per product), 0: the hi plane only (two)
  float scale_log2e;  // (1 / sqrt(head_dim)) * log2(e)
  int* status;
};

__global__ void __launch_bounds__(kAThreads, 1)
    sdpa_tc_kernel(const __grid_constant__ CUtensorMap tmap_k_hi,
                   const __grid_constant__ CUtensorMap tmap_k_lo,
                   const __grid_constant__ CUtensorMap tmap_vt_hi,
                   const __grid_constant__ CUtensorMap tmap_vt_lo, SdpaArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_v = base + kKSlots * kKPlane;   // the v^T ring follows the k ring
  uint8_t* book = smem + kARingBytes;
  // row maxima and row sums of the two softmax groups, then the barriers
  float* x_max = reinterpret_cast<float*>(book);          // [2][128]
  float* x_sum = reinterpret_cast<float*>(book + 1024);   // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(book + 2048);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_kfull = bar0;              // [4]  k ring: TMA bytes landed
  const uint32_t bar_kempty = bar0 + 32;        // [4]  k ring: slot read by its last MMA
  const uint32_t bar_sfull = bar0 + 64;         // [2]  scores of a block complete
  const uint32_t bar_pready = bar0 + 80;        // [2]  weights written over the scores
  const uint32_t bar_pvdone = bar0 + 96;        // [2]  P*V of a block complete
  const uint32_t bar_qready = bar0 + 112;       // Q planes in tensor memory
  const uint32_t bar_lready = bar0 + 120;       // both groups published their row sums
  const uint32_t bar_ofull = bar0 + 128;        // every MMA of the work item complete
  const uint32_t bar_vfull = bar0 + 136;        // [3]  v^T ring
  const uint32_t bar_vempty = bar0 + 160;       // [3]
  const uint32_t bar_pair = bar0 + 184;         // [4]  the two softmax warps that own the same 32 rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 27);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert(2048 + 27 * 8 + 8 <= kABookBytes, "book too small");

  if (base - raw > (uint32_t)kAAlignSlack) {
    // the dynamic shared memory starts further from a 1024-byte boundary than the launch
    // budgeted for: report it instead of running past the allocation
    if (threadIdx.x == 0) atomicCAS(g.status, 0, 0xb00 | 1);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = (int)((g.Lq + kBq - 1) / kBq);
  const int nblk = (int)((g.Lk + kBkv - 1) / kBkv);
  // the last block's second half of v^T is skipped when no key falls into it
  const int last_halves = g.Lk - (int64_t)(nblk - 1) * kBkv > kVKeys ? 2 : 1;
  const int num_items = nqt * g.heads;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kKSlots; i++) {
      mbar_init(bar_kfull + 8 * i, 1);
      mbar_init(bar_kempty + 8 * i, 1);
    }
    for (int i = 0; i < kVStages; i++) {
      mbar_init(bar_vfull + 8 * i, 1);
      mbar_init(bar_vempty + 8 * i, 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_pready + 8 * i, 8);
      mbar_init(bar_pvdone + 8 * i, 1);
    }
    for (int i = 0; i < 4; i++) mbar_init(bar_pair + 8 * i, 2);
    mbar_init(bar_qready, 8);
    mbar_init(bar_lready, 8);
    mbar_init(bar_ofull, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tmap_k_hi);
    prefetch_tmap(&tmap_k_lo);
    prefetch_tmap(&tmap_vt_hi);
    prefetch_tmap(&tmap_vt_lo);
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
      // ------------------------------------------------ TMA producer of k: a ring of four
      // slots of one plane (two boxes of 128 keys x 64 dims); a key block takes two (hi, then lo)
      const uint64_t keep = policy_evict_last();
      uint32_t slot = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int h = item / nqt;
        const int planes = g.k_lo ? 2 : 1;  // ring slots per key block
        for (int n = 0; n < planes * nblk; n++) {
          const int j = g.k_lo ? n >> 1 : n;
          const bool lo = g.k_lo && (n & 1);
          ok = mbar_wait(bar_kempty + 8 * slot, phase ^ 1u, abort_flag, g.status, 0x800 | 1);
          if (!ok) break;
          const uint32_t full = bar_kfull + 8 * slot;
          const uint32_t st = base + slot * kKPlane;
          mbar_expect_tx(full, kKPlane);
          for (int i = 0; i < 2; i++)
            tma_load_2d_hint(st + i * 16384, lo ? &tmap_k_lo : &tmap_k_hi, full, h * kHd + 64 * i, j * kBkv, keep);
          if (++slot == kKSlots) { slot = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 10) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer of v^T:
      // the two fp16 planes, one box of 128 dims x 64 keys each per stage
      const uint64_t keep = policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int h = item / nqt;
        const int nhalf = 2 * (nblk - 1) + last_halves;
        for (int j = 0; j < nhalf; j++) {
          ok = mbar_wait(bar_vempty + 8 * stage, phase ^ 1u, abort_flag, g.status, 0x800 | 3);
          if (!ok) break;
          const uint32_t full = bar_vfull + 8 * stage;
          const uint32_t st = smem_v + stage * kVStageBytes;
          mbar_expect_tx(full, g.v_lo ? kVStageBytes : kVPlane);
          tma_load_2d_hint(st, &tmap_vt_hi, full, j * kVKeys, h * kHd, keep);
          if (g.v_lo) tma_load_2d_hint(st + kVPlane, &tmap_vt_lo, full, j * kVKeys, h * kHd, keep);
          if (++stage == kVStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == 12) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuers of the scores: this lane
      // takes the blocks of one parity (warp 1 the even ones, warp 12 the odd ones), i.e. always
      // the same score buffer.  The k ring is shared: slot number `seq` of the CTA's whole run
      // is ring slot seq & 3, whose full barrier completes its phase (seq >> 2) & 1 for it.
      const uint32_t par = warp == 1 ? 0u : 1u;
      const uint32_t d2 = tmem_base + kColS + par * kBkv;
      uint32_t pv_ph = 0;                       // completed phases of pvdone[par]
      uint32_t q_ph = 0;
      uint32_t seq0 = 0;                        // k-ring sequence number of the item's first slot
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        // Q of this item is in tensor memory (written after every MMA of the previous item had
        // completed)
        ok = mbar_wait_spin(bar_qready, q_ph, abort_flag, g.status, 0x900 | 1);
        q_ph ^= 1u;
        if (!ok) break;
        tc_fence_after();
        // scores of this lane's blocks, three MMAs per 16 dims (the two small cross terms
        // first).  The buffer is free again when the P*V of the block two back has consumed its
        // weights; the k slots are released as soon as the scores that read them are done.
        bool any = false;
        for (int j = (int)par; j < nblk; j += 2) {
          const uint32_t seq = seq0 + (uint32_t)(g.k_lo ? 2 * j : j);
          const uint32_t slot_hi = seq & 3u, slot_lo = (seq + 1) & 3u;
          ok = mbar_wait_spin(bar_kfull + 8 * slot_hi, (seq >> 2) & 1u, abort_flag, g.status, 0x900 | 7);
          if (!ok) break;
          if (g.k_lo) {
            ok = mbar_wait_spin(bar_kfull + 8 * slot_lo, ((seq + 1) >> 2) & 1u, abort_flag, g.status, 0x900 | 6);
            if (!ok) break;
          }
          if (any) {
            ok = mbar_wait_spin(bar_pvdone + 8 * par, pv_ph, abort_flag, g.status, 0x900 | 8);
            if (!ok) break;
            pv_ph ^= 1u;
          }
          tc_fence_after();
          const uint32_t st_hi = base + slot_hi * kKPlane, st_lo = base + slot_lo * kKPlane;
#pragma unroll
          for (int ks = 0; ks < kHd / 16; ks++) {
            const uint32_t off = (uint32_t)((ks >> 2) * 16384);
            const uint64_t adv = (uint64_t)((ks & 3) * 2);
            const uint64_t k_hi = make_smem_desc(st_hi + off) + adv;
            const uint64_t k_lo = make_smem_desc(st_lo + off) + adv;
            umma_f16_ts(d2, tmem_base + kColQlo + ks * 8, k_hi, kIdescH, (uint32_t)(ks != 0));
            if (g.k_lo) umma_f16_ts(d2, tmem_base + kColQhi + ks * 8, k_lo, kIdescH, 1u);
            umma_f16_ts(d2, tmem_base + kColQhi + ks * 8, k_hi, kIdescH, 1u);
          }
          umma_commit(bar_kempty + 8 * slot_hi);
          if (g.k_lo) umma_commit(bar_kempty + 8 * slot_lo);
          umma_commit(bar_sfull + 8 * par);
          any = true;
        }
        if (!ok) break;
        if (any) {  // the completion of this lane's last block, so that the parity stays in step
          ok = mbar_wait_spin(bar_pvdone + 8 * par, pv_ph, abort_flag, g.status, 0x900 | 10);
          pv_ph ^= 1u;
          if (!ok) break;
        }
        seq0 += (uint32_t)(g.k_lo ? 2 * nblk : nblk);
      }
    }
  } else if (warp == 11) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuer of P*V
      uint32_t vstage = 0, vphase = 0;
      uint32_t pready_ph[2] = {0, 0};
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        // (O is free: every softmax warp read the previous item's O out before it could arrive
        // on this item's first pready)
        for (int j = 0; ok && j < nblk; j++) {
          const uint32_t buf = (uint32_t)(j & 1);
          ok = mbar_wait_spin(bar_pready + 8 * buf, pready_ph[buf], abort_flag, g.status, 0x900 | 9);
          if (!ok) break;
          pready_ph[buf] ^= 1u;
          const uint32_t pcol = tmem_base + kColS + buf * kBkv;
          const int halves = j == nblk - 1 ? last_halves : 2;
          for (int hf = 0; hf < halves; hf++) {
            ok = mbar_wait_spin(bar_vfull + 8 * vstage, vphase, abort_flag, g.status, 0x900 | 11);
            if (!ok) break;
            tc_fence_after();
            const uint32_t vt = smem_v + vstage * kVStageBytes;
#pragma unroll
            for (int ks = 0; ks < kVKeys / 16; ks++) {
              // 16 keys per instruction = 32 bytes of a v^T row: +2 in the address field.  The
              // weights of the block's keys 32c + 16i .. sit in 8 columns: hi at 32c + 8i, lo 16 further.
              const uint64_t v_hi = make_smem_desc(vt) + (uint64_t)(ks * 2);
              const uint64_t v_lo = make_smem_desc(vt + kVPlane) + (uint64_t)(ks * 2);
              const uint32_t p_hi = pcol + (uint32_t)((hf * 2 + (ks >> 1)) * 32 + (ks & 1) * 8);
              umma_f16_ts(tmem_base + kColO, p_hi + 16, v_hi, kIdescH, (uint32_t)((j | hf | ks) != 0));
              if (g.v_lo) umma_f16_ts(tmem_base + kColO, p_hi, v_lo, kIdescH, 1u);
              umma_f16_ts(tmem_base + kColO, p_hi, v_hi, kIdescH, 1u);
            }
            umma_commit(bar_vempty + 8 * vstage);
            if (++vstage == kVStages) { vstage = 0; vphase ^= 1u; }
          }
          if (!ok) break;
          umma_commit(bar_pvdone + 8 * buf);
        }
        if (!ok) break;
        umma_commit(bar_ofull);  // every P*V of the item (and so every MMA before them) is complete
      }
    }
  } else {
    // -------------------------------------------------- softmax groups + epilogue (8 warps)
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;        // 0: keys 0..63 of every block, 1: keys 64..127
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_col = tmem_base + kColS + (uint32_t)grp * 64 + lane_base;  // + buffer * kBkv
    const int sh_k = operand_shift(g.absmax[0]), sh_v = operand_shift(g.absmax[1]);
    uint32_t sfull_ph[2] = {0, 0};
    uint32_t pv_uses[2] = {0, 0};           // P*V completions on each score buffer before this item
    uint32_t l_ph = 0, ofull_ph = 0, pair_ph = 0;
    bool ok = true;
    // Meeting point of this warp and the one of the other group that owns the same rows (an
    // mbarrier like every other wait here, so that it is bounded): what either wrote to shared
    // memory before it is visible to the other after it.
    auto pair_sync = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pair + 8 * quarter);
      const bool r = mbar_wait_warp(bar_pair + 8 * quarter, pair_ph, abort_flag, g.status, 0xa00 | 7);
      pair_ph ^= 1u;
      return r;
    };
    for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      const int h = item / nqt, qt = item - h * nqt;
      const int64_t q0 = (int64_t)qt * kBq;
      const int64_t row = q0 + row_in_tile;
      // This thread's half of its query row (this group's 64 dims) -> registers; the row's
      // largest magnitude from both halves (the other one through shared memory) gives its
      // power of two; then fp16 hi and lo of q * 2^sh_q -> tensor memory, two elements per
      // column (zeros past Lq).
      const float* qhalf = g.q + row * g.C + (int64_t)h * kHd + grp * 64;
      float4 qv[16];
      uint32_t mx = 0;
#pragma unroll
      for (int j = 0; j < 16; j++) {
        qv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < g.Lq) qv[j] = *reinterpret_cast<const float4*>(qhalf + 4 * j);
      }
      {  // the next work item's rows on their way into L2 meanwhile
        const int nxt = item + (int)gridDim.x;
        if (nxt < num_items) {
          const int h2 = nxt / nqt, qt2 = nxt - h2 * nqt;
          const int64_t row2 = (int64_t)qt2 * kBq + row_in_tile;
          if (row2 < g.Lq) {
            const float* nq = g.q + row2 * g.C + (int64_t)h2 * kHd + grp * 64;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nq));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nq + 32));
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 16; j++)
        mx = max(max(mx, __float_as_uint(fabsf(qv[j].x))), max(__float_as_uint(fabsf(qv[j].y)),
                 max(__float_as_uint(fabsf(qv[j].z)), __float_as_uint(fabsf(qv[j].w)))));
      x_max[grp * kBq + row_in_tile] = __uint_as_float(mx);
      ok = pair_sync();
      if (!ok) break;
      mx = max(mx, __float_as_uint(x_max[(grp ^ 1) * kBq + row_in_tile]));
      const int sh_q = row < g.Lq ? operand_shift(mx) : 0;
      {
        const float qs = pow2f(sh_q);
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int j = 0; j < 16; j++) {
          split_f16x2(__fmul_rn(qv[j].x, qs), __fmul_rn(qv[j].y, qs), hi[2 * j], lo[2 * j]);
          split_f16x2(__fmul_rn(qv[j].z, qs), __fmul_rn(qv[j].w, qs), hi[2 * j + 1], lo[2 * j + 1]);
        }
        tmem_st_32x32(tmem_base + kColQhi + grp * 32 + lane_base, hi);
        tmem_st_32x32(tmem_base + kColQlo + grp * 32 + lane_base, lo);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_qready);
      }
      // scores arrive as (q 2^sh_q) . (k 2^sh_k): the factor that turns them into log2 units
      // (each factor a normal float; the product may round to zero or infinity only where the
      // reference's own scores leave the fp32 range)
      const float sc = __fmul_rn(__fmul_rn(g.scale_log2e, pow2f(-sh_q)), pow2f(-sh_k));
      // ---- one sweep over the keys with a running offset m_run per row (raw dot products):
      // weights p = 2^10 exp2((s - m_run) * sc).  The offset only moves when a block's maximum
      // exceeds it by more than kRescaleStep log2 units (the fp16 weights have room up to 2^15.8);
      // then O and the row sum are scaled down once, after the P*V that is still accumulating
      // into O has completed.  On ordinary data that happens in the first block or two of a row.
      float m_run = -INFINITY, e_off = 0.0f;
      float l = 0.0f;
      uint32_t hmax = 0;   // largest fp16 bit patterns of the weights' hi parts (two halves)
      for (int j = 0; j < nblk; j++) {
        const uint32_t buf = (uint32_t)(j & 1);
        ok = mbar_wait_warp(bar_sfull + 8 * buf, sfull_ph[buf], abort_flag, g.status, 0xa00 | 3);
        sfull_ph[buf] ^= 1u;
        if (!ok) break;
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(s_col + buf * kBkv, r0);
        tmem_ld_32x32(s_col + buf * kBkv + 32, r1);
        tmem_ld_wait();
        const int64_t key0 = (int64_t)j * kBkv + grp * 64;
        const int valid = (int)min((int64_t)64, g.Lk - key0);  // < 64 only in the last block
        // the block's maximum over this group's keys, then over the row's other 64 keys (the
        // thread of the other group that owns the same row), through shared memory
        float bm = -INFINITY;
        if (valid >= 64) {
#pragma unroll
          for (int t = 0; t < 32; t++) bm = fmaxf(bm, fmaxf(__uint_as_float(r0[t]), __uint_as_float(r1[t])));
        } else {
#pragma unroll
          for (int t = 0; t < 32; t++) {
            if (t < valid) bm = fmaxf(bm, __uint_as_float(r0[t]));
            if (32 + t < valid) bm = fmaxf(bm, __uint_as_float(r1[t]));
          }
        }
        float* xb = (j & 1) ? x_sum : x_max;          // alternating, so that one meeting per block is enough
        xb[grp * kBq + row_in_tile] = bm;
        ok = pair_sync();
        if (!ok) break;
        bm = fmaxf(bm, xb[(grp ^ 1) * kBq + row_in_tile]);
        const bool grow = __fmul_rn(__fsub_rn(bm, m_run), sc) > kRescaleStep;   // (true in the first block)
        if (__any_sync(0xffffffffu, grow)) {
          float f = 1.0f;
          if (grow) {
            if (j > 0) asm("ex2.approx.f32 %0, %1;" : "=f"(f) : "f"(__fmul_rn(__fsub_rn(m_run, bm), sc)));
            m_run = bm;
            e_off = __fsub_rn(kPShift, __fmul_rn(m_run, sc));
            l = __fmul_rn(l, f);
          }
          if (j > 0) {
            // O holds the blocks so far: the last P*V must have completed before O is scaled
            // (the next one waits for this block's weights).  The whole warp takes part in the
            // tensor-memory traffic; rows whose offset did not move scale by one.
            const uint32_t pb = (uint32_t)((j - 1) & 1);
            ok = mbar_wait_warp(bar_pvdone + 8 * pb, (pv_uses[pb] + (uint32_t)((j - 1) >> 1)) & 1u, abort_flag,
                                g.status, 0xa00 | 6);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 2 * grp; c < 2 * grp + 2; c++) {
              uint32_t o[32];
              tmem_ld_32x32(tmem_base + kColO + c * 32 + lane_base, o);
              tmem_ld_wait();
#pragma unroll
              for (int t = 0; t < 32; t++) o[t] = __float_as_uint(__fmul_rn(__uint_as_float(o[t]), f));
              tmem_st_32x32(tmem_base + kColO + c * 32 + lane_base, o);
            }
          }
        }
        // each 32 columns become: 16 columns of fp16 pairs p_hi, then 16 of p_lo.  The row sum
        // adds the weights themselves (they differ from hi + lo by 2^-22 at most).  A weight
        // beyond fp16's range (offset far too low) becomes an infinity that spoils only its own
        // row of O, and that row is marked for the fp32 pass by the test on hmax below.
        auto weights = [&](const uint32_t (&r)[32], int first, bool masked, uint32_t (&w)[32]) {
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            float p0, p1;
            const float e0 = __fmaf_rn(__uint_as_float(r[t]), sc, e_off);
            const float e1 = __fmaf_rn(__uint_as_float(r[t + 1]), sc, e_off);
            asm("ex2.approx.f32 %0, %1;" : "=f"(p0) : "f"(e0));
            asm("ex2.approx.f32 %0, %1;" : "=f"(p1) : "f"(e1));
            if (masked) {
              if (first + t >= valid) p0 = 0.0f;
              if (first + t + 1 >= valid) p1 = 0.0f;
            }
            l += __fadd_rn(p0, p1);
            uint32_t hi2, lo2;
            split_f16x2(p0, p1, hi2, lo2);
            hmax = __vmaxu2(hmax, hi2);
            w[t >> 1] = hi2;
            w[16 + (t >> 1)] = lo2;
          }
        };
        {
          uint32_t w[32];
          if (valid >= 64) {
            weights(r0, 0, false, w);
            tmem_st_32x32(s_col + buf * kBkv, w);
            weights(r1, 32, false, w);
            tmem_st_32x32(s_col + buf * kBkv + 32, w);
          } else {
            weights(r0, 0, true, w);
            tmem_st_32x32(s_col + buf * kBkv, w);
            weights(r1, 32, true, w);
            tmem_st_32x32(s_col + buf * kBkv + 32, w);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pready + 8 * buf);
      }
      if (!ok) break;
      pv_uses[0] += (uint32_t)((nblk + 1) >> 1);
      pv_uses[1] += (uint32_t)(nblk >> 1);
      ok = pair_sync();   // the partner has read this thread's last block maximum out of x_sum
      if (!ok) break;
      x_sum[grp * kBq + row_in_tile] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_lready);
      ok = mbar_wait_warp(bar_lready, l_ph, abort_flag, g.status, 0xa00 | 4);
      l_ph ^= 1u;
      if (!ok) break;
      l = x_sum[row_in_tile] + x_sum[kBq + row_in_tile];
      // head_dim * max|q_row| * max|k| bounds sum |q_d k_d|, here in log2 units of the weights
      const float bound = __fmul_rn(__fmul_rn(__uint_as_float(mx), __uint_as_float(g.absmax[0])),
                                    (float)kHd * g.scale_log2e);
      if (row < g.Lq && (max(hmax & 0xffffu, hmax >> 16) >= kPHalfTop || !(l >= kRowSumFloor) ||
                         !(bound <= kScoreBound)))
        g.redo[row * g.heads + h] = 1;   // offset too far from the row's maximum, or scores too large
      // O holds sum p 2^10 (v 2^sh_v): divide by the row sum of p 2^10 and take v's power back out
      const float inv = __fmul_rn(__fdiv_rn(1.0f, l), pow2f(-sh_v));
      // ---- epilogue: O / l, this group's two 32-column chunks, each thread its row's 128 bytes
      ok = mbar_wait_warp(bar_ofull, ofull_ph, abort_flag, g.status, 0xa00 | 5);
      ofull_ph ^= 1u;
      if (!ok) break;
      tc_fence_after();
      float* orow = g.out + row * g.C + (int64_t)h * kHd;
#pragma unroll 1
      for (int c = 2 * grp; c < 2 * grp + 2; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + kColO + c * 32 + lane_base, r);
        tmem_ld_wait();
        if (row < g.Lq) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            __stcs(reinterpret_cast<float4*>(orow + c * 32 + j),
                   make_float4(__fmul_rn(__uint_as_float(r[j]), inv), __fmul_rn(__uint_as_float(r[j + 1]), inv),
                               __fmul_rn(__uint_as_float(r[j + 2]), inv), __fmul_rn(__uint_as_float(r[j + 3]), inv)));
        }
      }
      // (the reads of O are complete: the next item's first pready arrival tells the P*V issuers)
      tc_fence_before();
    }
  }

  // ---------------------------------------------------- common exit
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);  // let bulk loads in flight land (~1 ms)
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// Largest magnitudes of k and of v (as fp32 bit patterns, which order like the magnitudes) into
// out[0] and out[1]; out starts at zero.
__global__ void __launch_bounds__(256) absmax_pair_kernel(const float* __restrict__ k,
                                                          const float* __restrict__ v, int64_t n,
                                                          uint32_t* __restrict__ out) {
  uint32_t mk = 0, mv = 0;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    mk = max(mk, __float_as_uint(fabsf(k[i])));
    mv = max(mv, __float_as_uint(fabsf(v[i])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mk = max(mk, __shfl_xor_sync(0xffffffffu, mk, o));
    mv = max(mv, __shfl_xor_sync(0xffffffffu, mv, o));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(out, mk);
    atomicMax(out + 1, mv);
  }
}

// k -> fp16 hi and lo planes of k * 2^sh (sh from the absmax pass).
__global__ void __launch_bounds__(256) split_planes_kernel(const float* __restrict__ x, int64_t n,
                                                           const uint32_t* __restrict__ absmax,
                                                           __half* __restrict__ hi,
                                                           __half* __restrict__ lo) {
  const float sc = pow2f(operand_shift(absmax[0]));
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float xs = __fmul_rn(x[i], sc);
    const __half h = __float2half_rn(xs);
    hi[i] = h;
    lo[i] = __float2half_rn(__fsub_rn(xs, __half2float(h)));
  }
}

// v [Lk, C] -> two fp16 planes of (v * 2^sh)^T, each [C, ld] (ld >= Lk, a multiple of 8; the
// padding is zero): hi = fp16(.), lo = fp16(. - hi).
__global__ void __launch_bounds__(256) transpose_split_f16_kernel(const float* __restrict__ v, int64_t Lk,
                                                                  int64_t C, int64_t ld,
                                                                  const uint32_t* __restrict__ absmax,
                                                                  __half* __restrict__ vt_hi,
                                                                  __half* __restrict__ vt_lo) {
  __shared__ float tile[32][33];
  const float sc = pow2f(operand_shift(absmax[1]));
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t k0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
  for (int r = ty; r < 32; r += 8)
    tile[r][tx] = (k0 + r < Lk && c0 + tx < C) ? v[(k0 + r) * C + c0 + tx] : 0.0f;
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    if (c0 + r < C && k0 + tx < ld) {
      const float x = __fmul_rn(tile[tx][r], sc);
      const __half h = __float2half_rn(x);
      const float rest = isfinite(x) ? __fsub_rn(x, __half2float(h)) : 0.0f;
      vt_hi[(c0 + r) * ld + k0 + tx] = h;
      vt_lo[(c0 + r) * ld + k0 + tx] = __float2half_rn(rest);
    }
  }
}

// Any head_dim / alignment: one warp per (query row, head), exact fp32 on the CUDA cores, three
// passes over the keys (maximum, sum, weighted values).  With `only`, just the marked rows.
__global__ void __launch_bounds__(256) sdpa_simt_kernel(const float* __restrict__ q,
                                                        const float* __restrict__ k,
                                                        const float* __restrict__ v, int64_t Lq,
                                                        int64_t Lk, int64_t C, int heads,
                                                        float scale, float* __restrict__ out,
                                                        const uint8_t* __restrict__ only) {
  const int lane = threadIdx.x & 31;
  const int64_t hd = C / heads;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t it = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); it < Lq * heads; it += warps) {
    if (only && !only[it]) continue;   // (marks are indexed like `it`: row * heads + head)
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

// v^T plane [C, ld] fp16, box = 128 rows x 64 keys (128 bytes), 128-byte swizzle.
bool make_tmap_vt(CUtensorMap* map, const void* ptr, int64_t C, int64_t Lk, int64_t ld, std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)Lk, (cuuint64_t)C};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kVKeys, (cuuint32_t)kHd};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(v^T) failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

// fp16 plane of k [Lk, C], box = 128 keys x 64 dims (128 bytes), 128-byte swizzle.
bool make_tmap_k(CUtensorMap* map, const void* ptr, int64_t Lk, int64_t C, std::string* why) {
  cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)Lk};
  cuuint64_t strides[1] = {(cuuint64_t)C * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)kBkv};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled(fp16 k plane) failed with CUresult " + std::to_string((int)r);
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

size_t sdpa_scratch_bytes(int64_t Lq, int64_t Lk, int64_t C, int heads) {
  const int64_t ld = (Lk + 7) / 8 * 8;
  // the two maxima; k and v^T hi, lo fp16; one mark per (query row, head)
  return 16 + (size_t)(2 * Lk * C + 2 * C * ld) * 2 + (size_t)(Lq * heads);
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
    sdpa_simt_kernel<<<(unsigned)blocks, 256, 0, s>>>(q, k, v, Lq, Lk, C, heads, scale, out, nullptr);
    return cudaGetLastError();
  }
  const int64_t ld = (Lk + 7) / 8 * 8;
  uint32_t* absmax = reinterpret_cast<uint32_t*>(scratch);
  __half* k_hi = reinterpret_cast<__half*>(scratch + 4);
  __half* k_lo = k_hi + Lk * C;
  __half* vt_hi = k_lo + Lk * C;
  __half* vt_lo = vt_hi + C * ld;
  uint8_t* redo = reinterpret_cast<uint8_t*>(vt_lo + C * ld);
  cudaError_t e = cudaMemsetAsync(absmax, 0, 16, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(redo, 0, (size_t)(Lq * heads), s);
  if (e != cudaSuccess) return e;
  int64_t blocks = (Lk * C + 255) / 256;
  if (blocks > (int64_t)sm_count * 16) blocks = (int64_t)sm_count * 16;
  count_launch(3);
  absmax_pair_kernel<<<(unsigned)blocks, 256, 0, s>>>(k, v, Lk * C, absmax);
  split_planes_kernel<<<(unsigned)blocks, 256, 0, s>>>(k, Lk * C, absmax, k_hi, k_lo);
  dim3 tgrid((unsigned)((C + 31) / 32), (unsigned)((ld + 31) / 32));
  transpose_split_f16_kernel<<<tgrid, 256, 0, s>>>(v, Lk, C, ld, absmax, vt_hi, vt_lo);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  CUtensorMap t_khi, t_klo, t_vt_hi, t_vt_lo;
  if (!make_tmap_k(&t_khi, k_hi, Lk, C, why) || !make_tmap_k(&t_klo, k_lo, Lk, C, why) ||
      !make_tmap_vt(&t_vt_hi, vt_hi, C, Lk, ld, why) || !make_tmap_vt(&t_vt_lo, vt_lo, C, Lk, ld, why))
    return cudaErrorInvalidValue;
  SdpaArgs g;
  g.v_lo = (flags & SDQ_SDPA_V_FP16) ? 0 : 1;
  g.k_lo = (flags & SDQ_SDPA_K_FP16) ? 0 : 1;
  g.q = q; g.out = out; g.absmax = absmax; g.redo = redo; g.Lq = Lq; g.Lk = Lk; g.C = C; g.heads = heads;
  g.scale_log2e = scale * 1.4426950408889634f;
  g.status = status;
  const int64_t items = ((Lq + kBq - 1) / kBq) * heads;
  count_launch();
  sdpa_tc_kernel<<<(unsigned)(items < sm_count ? items : sm_count), kAThreads, kASmemBytes, s>>>(
      t_khi, t_klo, t_vt_hi, t_vt_lo, g);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // rows whose offset was too far off (none on ordinary data): exact fp32 on the CUDA cores
  int64_t rblocks = (Lq * heads + 7) / 8;
  if (rblocks > (int64_t)sm_count * 8) rblocks = (int64_t)sm_count * 8;
  count_launch();
  sdpa_simt_kernel<<<(unsigned)rblocks, 256, 0, s>>>(q, k, v, Lq, Lk, C, heads, scale, out, redo);
  return cudaGetLastError();
}

}  // namespace sdq
