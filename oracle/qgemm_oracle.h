/*
 * CPU oracle for the int8 quantized-linear path.  TEST INFRASTRUCTURE ONLY:
 * the tests, the smoke check and the benchmark's CPU-baseline leg link this;
 * the product library never does.
 *
 * Every function restates, in plain C, the arithmetic of one piece of the
 * reference (JasonHonKL/Self-evolve-diffusion-cpp); the .c file cites the
 * reference file:line each one follows.  Parity status: PINNED -- the
 * restatement is checked bit-for-bit against the reference's own sd::qgemm /
 * sd::quantize_rowwise compiled from source (oracle/_ref) and against
 * tools/quantize/pack_sdcpp.py (fixtures under tests/golden/).
 */
#ifndef QGEMM_ORACLE_H
#define QGEMM_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* bf16 <-> f32 (src/core/tensor.cpp:39-47): RNE on the way down, <<16 up. */
void orc_f32_to_bf16(const float* src, uint16_t* dst, int64_t n);
void orc_bf16_to_f32(const uint16_t* src, float* dst, int64_t n);
/* IEEE binary16 -> f32, the packer's np.float16 -> np.float32 cast. */
void orc_f16_to_f32(const uint16_t* src, float* dst, int64_t n);

/* Dynamic per-row activation quantization (src/core/qgemm.cpp:82-96). */
void orc_act_quant_rows(const float* A, int64_t M, int64_t K, int8_t* aq, float* as);

/* s8 x s8 -> s32 accumulators, acc[i*N+j] = sum_k aq[i,k]*bq[j,k]
 * (src/core/qgemm.cpp:22-59; both M branches give the same sums). */
void orc_dot_s32(const int8_t* aq, const int8_t* bq, int64_t M, int64_t N, int64_t K,
                 int32_t* acc);

/* out = (float)acc * (as[i] * bs[j])   (src/core/qgemm.cpp:123-124,135). */
void orc_rescale(const int32_t* acc, const float* as, const float* bs, int64_t M, int64_t N,
                 float* out);

/* The whole sd::qgemm (src/core/qgemm.cpp:73-142). */
void orc_qgemm(const float* A, const int8_t* Bq, const float* bs, int64_t M, int64_t N,
               int64_t K, float* out);

/* y[i,j] += b[j]  (src/model/ovi_dit.cpp:71-79). */
void orc_bias_add(float* y, const float* b, int64_t M, int64_t N);

/* x[i,j] += y[i,j] * gate[j]  (gated_add_inplace, src/model/ovi_dit.cpp:152-159; one fused
 * multiply-add as in the reference's -O3 build) or, with gate NULL, x += y (add_inplace,
 * src/model/ovi_dit.cpp:144-149). */
void orc_residual_add(float* x, const float* y, const float* gate_or_null, int64_t M, int64_t N);

/* GELU, tanh form, in place (src/model/ovi_dit.cpp:132-142). */
void orc_gelu_tanh(float* x, int64_t n);

/* C++ weight quantizer sd::quantize_rowwise (src/core/tensor.cpp:63-78). */
void orc_quantize_rowwise(const float* W, int64_t N, int64_t K, int8_t* q, float* scale);

/* .sdcpp packer's quantizer quant_rows (tools/quantize/pack_sdcpp.py:45-51). */
void orc_quant_rows_packer(const float* x, int64_t rows, int64_t last, int8_t* q, float* scale);

/* w = q * scale[row]  (src/model/ovi_dit.cpp:53-63). */
void orc_dequant_rows(const int8_t* q, const float* scale, int64_t rows, int64_t last, float* w);

/* LayerNorm without affine parameters followed by the per-channel modulation
 * y = ln(x) * (1 + scale[c]) + shift[c]   (src/model/blocks.cpp:18-43 with w = b = null,
 * src/model/ovi_dit.cpp:162-173).  Sums run left to right in fp32 as the reference's do. */
void orc_layernorm_mod(const float* x, int64_t M, int64_t K, const float* shift,
                       const float* scale, float eps, float* y);

/* LayerNorm WITH its affine parameters, y = ln(x) * weight[c] + bias[c]
 * (src/model/blocks.cpp:18-43 with w, b given; call sites src/model/ovi_dit.cpp:241, :264). */
void orc_layernorm_affine(const float* x, int64_t M, int64_t K, const float* weight,
                          const float* bias, float eps, float* y);

/* sd::matmul, portable branch (src/core/gemm.cpp:100-110, 33-40): fp32 sums left to right,
 * w is [K,N] row-major.  Tolerance-level comparisons only (the reference's SIMD / BLAS branches
 * add in other orders). */
void orc_matmul_f32(const float* a, int64_t M, int64_t K, const float* w, int64_t N,
                    const float* bias_or_null, float* out);

/* blk::sdpa (src/model/blocks.cpp:113-199): out[Lq,C] = softmax(q k^T / sqrt(C/heads)) v per head,
 * q [Lq,C], k and v [Lk,C], fp32, no mask.  Tolerance-level comparisons only (expf and the
 * summation orders differ between builds). */
void orc_sdpa(const float* q, const float* k, const float* v, int64_t Lq, int64_t Lk, int64_t C,
              int heads, float* out);

/* Threads used by the loops above; <=0 restores the default. */
void orc_set_threads(int n);
int orc_threads(void);

#ifdef __cplusplus
}
#endif
#endif
