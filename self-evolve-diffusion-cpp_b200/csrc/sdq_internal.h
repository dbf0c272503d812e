// Internal declarations shared by the translation units of libsdq.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "sdq.h"

namespace sdq {

// ---- error plumbing (sdq_api.cu) ----
int fail(int code, const std::string& msg);  // records msg for sdq_last_error, returns code
int cuda_fail(cudaError_t e, const char* what);
#define SDQ_CUDA(expr)                                             \
  do {                                                             \
    cudaError_t _e = (expr);                                       \
    if (_e != cudaSuccess) return ::sdq::cuda_fail(_e, #expr);     \
  } while (0)

void count_launch(int n = 1);

// ---- activation / weight quantization kernels (quant_kernels.cu) ----
// aq int8 [M,K], a_scale f32 [M]; all device pointers.
cudaError_t launch_act_quant(const float* A, int64_t M, int64_t K, int8_t* aq, float* a_scale,
                             int sm_count, cudaStream_t s);
// LayerNorm (no affine) + modulation + activation quantization; h_out (fp32 [M,K]) optional.
// With `stats` (scratch, M float2) a first kernel computes each row's mean and 1/sqrt(var+eps)
// with the reference's left-to-right sums and the result is bit-identical to the CPU's; with
// stats null the sums are block-wide trees (one kernel, one pass, equal to rounding error).
// affine != 0: `scale` / `shift` are the layernorm's own weight and bias, h = ln * w + b.
// cudaErrorInvalidValue when K % 4 != 0, K > 16384 or a pointer is not 16-byte aligned.
cudaError_t launch_ln_mod_quant(const float* X, int64_t M, int64_t K, const float* shift,
                                const float* scale, float eps, int8_t* aq, float* a_scale,
                                float* h_out, float2* stats, int affine, int sm_count,
                                cudaStream_t s);
// src_dtype SDQ_F32/BF16/F16, mode SDQ_MODE_*; all device pointers.
cudaError_t launch_quantize_rows(const void* src, int src_dtype, int64_t rows, int64_t last,
                                 int mode, int8_t* q, float* scale, int sm_count, cudaStream_t s);
cudaError_t launch_dequant_rows(const int8_t* q, const float* scale, int64_t rows, int64_t last,
                                float* w, int sm_count, cudaStream_t s);

// ---- GEMM kernels ----
struct GemmArgs {
  const int8_t* aq;       // [M,K]
  const float* a_scale;   // [M]
  const int8_t* bq;       // [N,K]
  const float* b_scale;   // [N]
  const float* bias;      // [N] or null
  float* out;             // [M,N]
  int32_t* acc_dump;      // [M,N] or null
  int64_t M, N, K;
  uint32_t flags;         // SDQ_GELU_TANH
  int* status;            // device word: 0 ok, else a code written by a kernel that gave up
  // Column-split multi-GPU form: this launch computes columns [out_col0, out_col0 + N) of a
  // wider [M, out_ld] result and writes the block into out_copies buffers (this GPU's and
  // its peers').  out_copies == 0 is the ordinary single-output case (out, row pitch N).
  int64_t out_col0 = 0, out_ld = 0;
  int out_copies = 0;
  float* out_all[8] = {};
  // Residual epilogue: out = residual + y * gate[j] (gate null: residual + y), y being the
  // value the epilogue would otherwise store.  residual is fp32 [M,N] and may be `out` itself.
  const float* residual = nullptr;
  const float* gate = nullptr;    // [N] or null; only read when residual is set
  int32_t* splitk_acc = nullptr;  // [M,N] zeroed int32 sums when K is split, else null
  int k_splits = 1;               // >1 only together with splitk_acc
  // 2-CTA kernel: all-zero int32 scratch of tail_cap_tiles x 256 x 256 for the partial sums of
  // the last, partial wave's tiles (null: every tile is computed by one CTA pair).  The launch
  // leaves it all zero again.  Filled in by the caller; the launcher decides whether to use it.
  int32_t* tail_acc = nullptr;
  int tail_cap_tiles = 0;
  // 2-CTA kernel, set by the launcher: height of a band of the tile walk in 256-row pairs, and
  // the L2 eviction classes of the operand loads (see launch_qgemm_tc2).
  int group_pairs = 0;
  int a_policy = 0, b_policy = 0;
};


// The bulk-store epilogues of the tcgen05 kernels read b_scale, bias and gate four floats at a
// time: true when those pointers allow it (16-byte aligned).  Otherwise the per-thread scalar
// epilogue has to be used.
inline bool epilogue_vectors_aligned(const GemmArgs& g) {
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return aligned(g.b_scale) && (!g.bias || aligned(g.bias)) &&
         (!g.residual || !g.gate || aligned(g.gate));
}

// Portable CUDA-core kernel (any M, N, K): qgemm_simt.cu
cudaError_t launch_qgemm_simt(const GemmArgs& g, cudaStream_t s);

// tcgen05 kernel: qgemm_tcgen05.cu.  Needs K % 16 == 0 and 16-byte aligned aq / bq.
bool qgemm_tc_supported(const GemmArgs& g);
// Returns cudaSuccess or the launch error; `why` receives text on tensor-map failures.
cudaError_t launch_qgemm_tc(const GemmArgs& g, int sm_count, cudaStream_t s, std::string* why);
// K slices the planner wants for this problem (1 = none); the caller then provides a
// zeroed [M,N] int32 accumulator in g.splitk_acc and sets g.k_splits to this value.
int qgemm_tc_plan_splits(const GemmArgs& g, int sm_count);
// One-time set-up (driver entry point lookup, max-shared-memory attributes).
int qgemm_tc_setup(std::string* why);

// 2-CTA (cta_group::2) variant for large problems: qgemm_tcgen05_2cta.cu.
int qgemm_tc2_setup(std::string* why);
bool qgemm_tc2_wanted(const GemmArgs& g, int sm_count);  // call only if qgemm_tc_supported(g)
// Tiles of the last, partial wave the 2-CTA launcher would share between all CTA pairs if
// GemmArgs::tail_acc holds that many zeroed 256 x 256 int32 tiles (0: no scratch needed).
int qgemm_tc2_tail_tiles(const GemmArgs& g, int sm_count);
// Why the 2-CTA kernel cannot take this problem at all (null: it can).
const char* qgemm_tc2_unfit(const GemmArgs& g);
cudaError_t launch_qgemm_tc2(const GemmArgs& g, int sm_count, cudaStream_t s, std::string* why);

// ---- fp32 matmul on tcgen05, three tf32 products per fp32 product: fgemm_tcgen05.cu ----
int fgemm_setup(std::string* why);
// W [K,N] fp32 row-major (device) -> tf32 planes hi / lo, transposed to [N,K].
cudaError_t launch_transpose_split(const float* w_kn, int64_t K, int64_t N, float* hi_nk, float* lo_nk,
                                   cudaStream_t s);
// out[M,N] = a[M,K] * W + bias.  a_hi / a_lo: scratch planes of M*K floats each (unused by the
// CUDA-core path taken when K % 4 != 0, a pointer is unaligned or SDQ_FORCE_SIMT is set).
cudaError_t launch_fmatmul(const float* a, int64_t M, int64_t K, const float* w_hi, const float* w_lo,
                           int64_t N, const float* bias, float* out, float* a_hi, float* a_lo,
                           int* status, uint32_t flags, int sm_count, cudaStream_t s, std::string* why);

// ---- exact-softmax attention (blk::sdpa) on tcgen05: sdpa_tcgen05.cu ----
int sdpa_setup(std::string* why);
size_t sdpa_scratch_bytes(int64_t Lq, int64_t Lk, int64_t C, int heads);  // fp16 planes of k and v^T, per-row redo marks
// out[Lq,C] = softmax(q k^T / sqrt(C/heads)) v per head; q [Lq,C], k and v [Lk,C], all device fp32.
cudaError_t launch_sdpa(const float* q, const float* k, const float* v, int64_t Lq, int64_t Lk,
                        int64_t C, int heads, float* out, float* scratch, int* status,
                        uint32_t flags, int sm_count, cudaStream_t s, std::string* why);

// MMA-issue-bound int8 rate of the device (mma_probe.cu).
int int8_mma_probe(int sm_count, int iters, int* status_dev, double* seconds, double* ops);
int wait_expiry_selftest(int limit_ms, int code, int* status_dev, int* outcome_dev, cudaStream_t s);

}  // namespace sdq
