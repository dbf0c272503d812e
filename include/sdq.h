/*
 * sdq -- C ABI of the B200 (sm_100a) int8 quantized-linear path.
 *
 * This is the boundary a host program binds to replace the CPU implementation
 * of the int8 linear in JasonHonKL/Self-evolve-diffusion-cpp: dynamic per-row
 * int8 activation quantization + s8 x s8 -> s32 GEMM + fp32 rescale
 * (sd::qgemm), the two weight quantizers, and the .sdcpp pack reader/writer.
 * Plain pointers and sizes only; every function returns an sdq_status and the
 * text of the last failure on the calling thread is in sdq_last_error().
 *
 * One process drives one GPU: call sdq_init(device) first.  There is no CPU
 * fallback: without a usable sm_100 device every compute entry point fails
 * with SDQ_ERR_CUDA / SDQ_ERR_NOT_INIT.
 *
 * Each declaration cites the reference interface it replaces (file:line in
 * the reference project).
 */
#ifndef SDQ_H
#define SDQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SDQ_VERSION 1

#if defined(__GNUC__)
#define SDQ_API __attribute__((visibility("default")))
#else
#define SDQ_API
#endif

typedef enum sdq_status {
  SDQ_OK = 0,
  SDQ_ERR_INVALID = 1,        /* bad argument (null pointer, negative size, wrong handle) */
  SDQ_ERR_CUDA = 2,           /* a CUDA runtime/driver call failed */
  SDQ_ERR_NOT_INIT = 3,       /* sdq_init has not succeeded in this process */
  SDQ_ERR_IO = 4,             /* file cannot be opened / read / written / mapped */
  SDQ_ERR_FORMAT = 5,         /* malformed .sdcpp or .safetensors content */
  SDQ_ERR_DEVICE_TIMEOUT = 6, /* a bounded wait inside a kernel gave up; output is invalid */
  SDQ_ERR_NOT_FOUND = 7,
  SDQ_ERR_NOMEM = 8
} sdq_status;

/* Opaque handle of an int8 weight matrix [N,K] + fp32 scales [N] resident in HBM. 0 = none. */
typedef uint64_t sdq_weight_t;

/* ---- flags of the compute entry points ---- */
#define SDQ_A_HOST 0x1u      /* A is host memory: it is copied to the device inside the call */
#define SDQ_OUT_HOST 0x2u    /* out is host memory: the result is copied back inside the call */
#define SDQ_GELU_TANH 0x4u   /* apply GELU (tanh form) after the bias in the epilogue */
#define SDQ_FORCE_SIMT 0x8u  /* use the portable CUDA-core kernel instead of tcgen05 */
#define SDQ_SYNC 0x10u       /* wait for the stream before returning */
#define SDQ_LN_TREE_SUMS 0x20u /* layernorm mean/variance as block-wide tree sums (one pass over
                                  x, equal to the CPU to rounding error) instead of the
                                  reference's left-to-right sums (bit-identical, two more passes) */

#define SDQ_LN_AFFINE 0x40u  /* sdq_layernorm_mod_quantize: `scale` and `shift` are the layernorm's
                                own weight and bias, h = ln * weight + bias */
#define SDQ_SDPA_V_FP16 0x80u /* sdq_sdpa: v enters P*V as one fp16 number per element (11 mantissa
                               * bits, after its power-of-two scaling) instead of two: two MMAs per
                               * product instead of three and half the v^T traffic; outputs move by
                               * up to ~2.5e-4 of the largest (inside the reference's 1e-3 bound) */

#define SDQ_SDPA_K_FP16 0x100u /* sdq_sdpa: k enters the scores as one fp16 number per element (q keeps
                                * both of its planes): two MMAs per product instead of three and half the
                                * k traffic.  The scores then carry k's 2^-12 rounding, which the softmax
                                * turns into a relative error of the same size on every weight; see the
                                * measured figures beside SDQ_SDPA_V_FP16 in the description of sdq_sdpa */

/* source element types of sdq_quantize_rows (the packer's SRC table,
 * tools/quantize/pack_sdcpp.py:26-35) */
#define SDQ_F32 0
#define SDQ_BF16 1
#define SDQ_F16 2

/* rounding recipe of sdq_quantize_rows */
#define SDQ_MODE_PACKER 0  /* quant_rows, tools/quantize/pack_sdcpp.py:45-51 */
#define SDQ_MODE_ROWWISE 1 /* sd::quantize_rowwise, src/core/tensor.cpp:63-78 */

#define SDQ_SRC_HOST 0x1u /* sdq_quantize_rows / sdq_dequant_rows: src is host memory */
#define SDQ_DST_HOST 0x2u /* ... q/scale (or w) are host memory */

/* ---- process / device ---- */

/* Binds this process to CUDA device `device` and creates the context state
 * (replaces nothing in the reference: it has no device).  Idempotent for the
 * same device. */
SDQ_API int sdq_init(int device);
SDQ_API int sdq_shutdown(void);
SDQ_API int sdq_device(void); /* -1 before sdq_init */
SDQ_API int sdq_version(void);
SDQ_API const char* sdq_last_error(void);
/* Number of kernels this library has launched since sdq_init (monotonic). */
SDQ_API int64_t sdq_launch_count(void);

/* A measuring stick (no counterpart in the reference): every SM issues `iters` batches of 16
 * tcgen05.mma kind::i8 (M=128, N=256, K=32) back to back on operands already in shared memory
 * -- no TMA, no epilogue, no global traffic.  Returns the device time of the launch and the
 * rate in TOPS: the MMA-issue-bound int8 ceiling of this GPU at the clocks it holds, which
 * is what the GEMM kernels' tensor rooflines are compared with.  Synchronous. */
SDQ_API int sdq_int8_mma_probe(int iters, double* seconds, double* tera_ops_per_s);

/* Self-test of the time-out path (no counterpart in the reference).  Launches, on `stream`, one
 * warp that waits -- through the bounded wait every tensor-core kernel of the library uses -- on
 * a barrier nothing ever arrives on, with a limit of `limit_ms` milliseconds (1..1000) instead of
 * the kernels' 2 s.  The wait runs out, the kernel records SDQ_SELFTEST_WAIT_CODE in the
 * library's status word, raises its abort flag and returns; *outcome_dev (device memory)
 * receives bit 0 = "the wait was satisfied" (never), bit 1 = "the abort flag was seen raised".
 * Asynchronous: the next sdq_stream_sync (or SDQ_SYNC call) returns SDQ_ERR_DEVICE_TIMEOUT
 * naming the code, exactly once; the context stays usable and later calls are unaffected.
 * Nothing hangs or faults: the kernel ends by itself a few milliseconds after the limit. */
#define SDQ_SELFTEST_WAIT_CODE 0x7e01
SDQ_API int sdq_selftest_wait_expiry(int limit_ms, int* outcome_dev, void* stream);

/* Device / pinned-host memory and copies for callers that do not link the CUDA
 * runtime themselves.  `stream` is a cudaStream_t (NULL = default stream). */
SDQ_API int sdq_malloc(void** dptr, size_t bytes);
SDQ_API int sdq_free(void* dptr);
SDQ_API int sdq_malloc_host(void** hptr, size_t bytes);
SDQ_API int sdq_free_host(void* hptr);
SDQ_API int sdq_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
SDQ_API int sdq_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
SDQ_API int sdq_memset(void* dst, int value, size_t bytes, void* stream);
SDQ_API int sdq_stream_sync(void* stream);
/* A new non-blocking stream / its destruction, for callers without the CUDA runtime.  The
 * scratch of the compute entry points is kept per stream: calls on different streams may run
 * concurrently (also from different host threads); concurrent calls on ONE stream may not. */
SDQ_API int sdq_stream_create(void** stream);
SDQ_API int sdq_stream_destroy(void* stream);

/* ---- weights ---- */

/* Copies one packed weight -- int8 [N,K] row-major (torch Linear [out,in], the
 * layout sd::qgemm takes as Bq, src/core/tensor.h:48-52) and its N fp32 scales
 * -- into 256-byte-aligned device memory, once, and remembers the host address
 * so that sdq_weight_lookup(q_host) finds it again.  The host pointers may have
 * any alignment (the .sdcpp blob has no padding, src/serde/sdcpp.cpp:107-124). */
SDQ_API int sdq_weight_upload(const int8_t* q_host, const float* scale_host, int64_t N, int64_t K,
                      sdq_weight_t* out);
/* Wraps device-resident int8 weights without copying (caller keeps them alive). */
SDQ_API int sdq_weight_wrap_device(const int8_t* q_dev, const float* scale_dev, int64_t N, int64_t K,
                           sdq_weight_t* out);
/* Finds the weight uploaded from host address `q_host` (the key the reference's
 * caller has in hand: blk::Linear::w.data, src/model/ovi_dit.cpp:66-70). */
SDQ_API int sdq_weight_lookup(const void* q_host, sdq_weight_t* out);
/* Extents and device addresses of a weight; for an fp32 weight (sdq_fweight_upload) q_dev and
 * scale_dev are reported as NULL.  Any out pointer may be NULL. */
SDQ_API int sdq_weight_info(sdq_weight_t w, int64_t* N, int64_t* K, const int8_t** q_dev,
                    const float** scale_dev);
SDQ_API int sdq_weight_release(sdq_weight_t w);

/* ---- the hot path ---- */

/* out[M,N] = qgemm(A[M,K], W)  -- replaces sd::qgemm (src/core/tensor.h:52,
 * src/core/qgemm.cpp:73-142): per-row absmax int8 quantization of the fp32
 * activations, s8 x s8 -> s32 dot products against the weight rows, then
 * out = (float)acc * (a_scale[i] * w_scale[j]).  `bias` (fp32 [N], device
 * memory, may be NULL) fuses the y[i,j] += b[j] pass the reference's caller
 * runs afterwards (src/model/ovi_dit.cpp:71-79); SDQ_GELU_TANH fuses the
 * activation between the two FFN linears (src/model/ovi_dit.cpp:132-142,
 * 214-222).  A and out are device memory unless SDQ_A_HOST / SDQ_OUT_HOST.
 * M == 0 is a no-op (src/core/qgemm.cpp:76); a weight always has N >= 1 and K >= 1.
 * Like the reference (src/core/qgemm.cpp:21), the int32 sums cannot overflow for K <= 133152.
 * Alignment: fp32 pointers need only their natural 4 bytes.  The fast epilogue (bulk tensor
 * stores, scales / bias / gate read four at a time) is taken when out, the weight's scales,
 * bias, gate and residual are 16-byte aligned and N % 4 == 0; anything else -- a bias that is a
 * slice of a larger vector at an odd offset, say -- runs the per-element epilogue of the 1-CTA
 * kernel, same bits, slower.  This holds for every entry point that takes these pointers
 * except sdq_qgemm_colsplit, which has only the fast form and rejects such pointers. */
SDQ_API int sdq_qgemm(sdq_weight_t w, const float* A, int64_t M, float* out, const float* bias,
              uint32_t flags, void* stream);

/* First half of sd::qgemm alone (src/core/qgemm.cpp:82-96): aq int8 [M,K] and
 * a_scale fp32 [M], all device memory. */
SDQ_API int sdq_quantize_activations(const float* A_dev, int64_t M, int64_t K, int8_t* aq_dev,
                             float* a_scale_dev, void* stream);

/* The step the reference runs in front of most DiT linears, fused with the first half of
 * sd::qgemm: LayerNorm without affine parameters (blk::layernorm, src/model/blocks.cpp:18-43),
 * the per-channel modulation h = ln * (1 + scale[c]) + shift[c] (mod_rows,
 * src/model/ovi_dit.cpp:162-173; call sites :205-217) and the activation quantization
 * (src/core/qgemm.cpp:82-96): fp32 `h` is never written unless `h_out_dev` (fp32 [M,K], may be
 * NULL) asks for it.  Feed aq / a_scale to sdq_qgemm_prequantized.
 * By default the row mean and variance are the reference's own left-to-right fp32 sums (a
 * first kernel runs one row per lane through the same chain of additions), the modulation is
 * the single fused multiply-add of the reference's -O3 build, and h, aq and a_scale are
 * bit-identical to the CPU's.  With SDQ_LN_TREE_SUMS the sums are block-wide trees in the same
 * pass as everything else: about twice as fast for this step, h equal to rounding error, and an
 * int8 value may differ by one step where h lands on a rounding boundary.
 * With SDQ_LN_AFFINE the same kernels serve the layernorm that HAS parameters, in front of the
 * cross-attention projections (src/model/ovi_dit.cpp:241, :264): scale_dev is its weight and
 * shift_dev its bias, h = ln * weight + bias (one fused multiply-add, as in the reference's build).
 * K % 4 == 0, K <= 16384, pointers 16-byte aligned. */
SDQ_API int sdq_layernorm_mod_quantize(const float* X_dev, int64_t M, int64_t K,
                                       const float* shift_dev, const float* scale_dev, float eps,
                                       int8_t* aq_dev, float* a_scale_dev, float* h_out_dev,
                                       uint32_t flags, void* stream);

/* Second half of sd::qgemm (src/core/qgemm.cpp:98-138) on activations that are
 * already quantized: lets a caller quantize x once and run the q, k and v
 * projections on it (the reference re-quantizes x three times,
 * src/model/ovi_dit.cpp:176-188).  `acc_dump_dev` (int32 [M,N], may be NULL)
 * also receives the raw s32 accumulators. */
SDQ_API int sdq_qgemm_prequantized(sdq_weight_t w, const int8_t* aq_dev, const float* a_scale_dev,
                           int64_t M, float* out_dev, const float* bias_dev,
                           int32_t* acc_dump_dev, uint32_t flags, void* stream);

/* ---- one linear split by output columns over the GPUs of a box ----
 * No counterpart in the reference (it is single-process CPU code); columns of sd::qgemm's
 * output are independent (each weight row has its own scale, src/core/qgemm.cpp:123-135), so
 * a rank that holds weight rows [col0, col0+Nw) computes out[:, col0:col0+Nw] exactly.
 * sdq_qgemm_colsplit fuses the exchange into the GEMM: the epilogue writes the finished
 * block straight into `n_outs` destination buffers, each a full [M, N_total] fp32 matrix --
 * this GPU's own and its peers' (addresses from sdq_ipc_open; the stores cross NVLink).
 * When every rank has made the call and the ranks have synchronised (any barrier after the
 * stream work), every buffer holds the complete row-major result: an all-gather without a
 * separate collective or re-layout pass.  col0 must be a multiple of 32 and Nw a multiple
 * of 32 unless the block is the last one; N_total % 4 == 0; destinations 16-byte aligned.
 * sdq_ipc_export/open/close exchange buffers made by sdq_malloc between the processes
 * (64-byte CUDA IPC handles, carried by whatever channel the host program has). */
SDQ_API int sdq_qgemm_colsplit(sdq_weight_t w_block, const float* A_dev, int64_t M, int64_t col0,
                               int64_t N_total, float* const* outs_dev, int n_outs,
                               const float* bias_block_dev, uint32_t flags, void* stream);
SDQ_API int sdq_ipc_export(const void* dptr, unsigned char handle[64]);
SDQ_API int sdq_ipc_open(const unsigned char handle[64], void** dptr);
SDQ_API int sdq_ipc_close(void* dptr);

/* y = fc2(gelu_tanh(fc1(x))) for one FFN -- replaces the three lines of the reference's
 * ffn_fwd that are on this path (src/model/ovi_dit.cpp:218-220: mlin fc1,
 * gelu_tanh_inplace, mlin fc2; each mlin = sd::qgemm + bias pass).  x is fp32
 * [M, K1], y fp32 [M, N2]; w2's K must equal w1's N.  Device pointers by default;
 * `hidden_dev` (fp32 [M, N1], device, may be NULL) receives the activations between
 * the two linears.  With SDQ_A_HOST | SDQ_OUT_HOST (both or neither) x and y are host
 * memory -- pinned memory makes the copies asynchronous -- and the rows are processed
 * in chunks so that the upload of the next chunk and the download of the previous one
 * overlap the arithmetic; hidden_dev is ignored and the call returns when y is complete. */
SDQ_API int sdq_ffn_pair(sdq_weight_t w1, const float* bias1_dev, sdq_weight_t w2,
                         const float* bias2_dev, const float* x, int64_t M, float* hidden_dev,
                         float* y, uint32_t flags, void* stream);

/* A linear followed by the residual update its caller in the reference runs as separate
 * passes over [M,N]:  out = residual + (qgemm(A, W) + bias) * gate[j].
 * With `gate_dev` (fp32 [N]) this is mlin + gated_add_inplace (src/model/ovi_dit.cpp:66-84,
 * 152-159; call sites :205-212 and :214-222); with gate_dev NULL it is mlin + add_inplace
 * (:144-149; call sites :254-255 and :266-267).  `residual_dev` is fp32 [M,N] and may be
 * `out_dev` itself (the reference updates x in place).  The multiply-add is ONE fused
 * operation, as in the reference built by its own Makefile (-O3 on an FMA target; checked
 * against the compiled function), so the result is bit-identical to that build.  Device
 * pointers only. */
SDQ_API int sdq_qgemm_residual(sdq_weight_t w, const float* A_dev, int64_t M,
                               const float* residual_dev, const float* gate_dev, float* out_dev,
                               const float* bias_dev, uint32_t flags, void* stream);

/* The whole ffn_fwd of a DiT block (src/model/ovi_dit.cpp:214-222), in place on x fp32 [M,D]:
 *   h = layernorm(x) * (1 + scale) + shift;  y = fc2(gelu_tanh(fc1(h)));  x += y * gate
 * as four launches: layernorm + modulation + quantization fused (sdq_layernorm_mod_quantize),
 * fc1 + bias + GELU, quantization, fc2 + bias + gated residual.  shift / scale / gate are
 * fp32 [D] (rows 3, 4, 5 of the block's modulation table).  Everything is bit-identical to
 * the CPU's except the GELU (the device's ex2/rcp against libm's tanh), so x matches the CPU
 * within the 1e-3 bound; SDQ_LN_TREE_SUMS in `flags` trades the exact layernorm sums for one
 * pass less over x.  D % 4 == 0, D <= 16384; device pointers only. */
SDQ_API int sdq_ffn_block(sdq_weight_t w1, const float* bias1_dev, sdq_weight_t w2,
                          const float* bias2_dev, float* x_dev, int64_t M, const float* shift_dev,
                          const float* scale_dev, const float* gate_dev, float eps, uint32_t flags,
                          void* stream);

/* ---- the fp32 linears beside the int8 ones ----
 * out[M,N] = A[M,K] * W[K,N] + bias  -- replaces sd::matmul (src/core/tensor.h:46,
 * src/core/gemm.cpp:115-160) as blk::linear calls it (src/model/blocks.cpp:13-16) for the
 * tensors a pack keeps in fp32 (numel < 65536 or --dtype-preserve) and for unpacked
 * checkpoints.  W is the reference's Linear layout, fp32 [K = in, N = out] row-major;
 * sdq_fweight_upload (SDQ_A_HOST: `w` is host memory, else device) transposes it once into
 * [N,K] and splits it into two tf32 planes.  sdq_fmatmul issues three tf32 tensor-core products
 * per fp32 product (hi*hi + hi*lo + lo*hi, K accumulated in groups of 256 that are added in
 * fp32 registers): about 2e-6 of the largest output, the level of an fp32 BLAS, for any K.
 * The reference's own sums depend on its BLAS / SIMD order, so this path is held to
 * the reference's matmul tolerance (max-abs error <= 1e-3 of the largest output,
 * tests/test_core.cpp:82-84), not to bit equality.  The handle is released with
 * sdq_weight_release; the int8 entry points reject it and vice versa.  A / out are device
 * memory unless SDQ_A_HOST / SDQ_OUT_HOST; bias is device memory or NULL. */
SDQ_API int sdq_fweight_upload(const float* w, int64_t K, int64_t N, uint32_t flags,
                               sdq_weight_t* out);
SDQ_API int sdq_fmatmul(sdq_weight_t w, const float* A, int64_t M, float* out,
                        const float* bias_dev, uint32_t flags, void* stream);

/* ---- attention between the projections ----
 * out[Lq,C] = softmax(q k^T / sqrt(C/heads)) v for each of `heads` heads -- replaces blk::sdpa
 * (src/model/blocks.h:60-66, src/model/blocks.cpp:113-199; the reference never sets its causal
 * flag).  q is fp32 [Lq,C], k and v fp32 [Lk,C], all device memory; head h owns columns
 * [h*C/heads, (h+1)*C/heads).  For head_dim 128 (the DiT's) everything runs on the tensor
 * cores: q, k, v and the softmax weights are each carried as two fp16 numbers times a power of
 * two (22 mantissa bits; the powers are found from the data, so magnitudes do not matter), every
 * product is three fp16 MMAs with fp32 accumulation, in one sweep over the keys with a running
 * offset per row (the accumulator is rescaled only when a row's maximum moves by more than 4
 * log2 units, i.e. in its first blocks).  Rows whose scores are out of that
 * scheme's range (|score| in the tens of thousands) are recomputed in plain fp32 by the CUDA-core
 * kernel that also serves the other head sizes.  Held to the reference's 1e-3 bound (max-abs
 * error / max-abs output; ~1e-5 measured at a few thousand keys, 1e-4 at 27280; flags may carry
 * SDQ_SDPA_V_FP16, SDQ_FORCE_SIMT, SDQ_SYNC); exp and the
 * summation order are not bit-identical to the CPU's, but two runs give the same bits. */
SDQ_API int sdq_sdpa(const float* q_dev, const float* k_dev, const float* v_dev, int64_t Lq,
                     int64_t Lk, int64_t C, int heads, float* out_dev, uint32_t flags,
                     void* stream);

/* The same computation as sdq_qgemm for callers that cannot allocate device memory
 * while they run (a host that has given all HBM to its own pool, a plugin inside
 * another allocator, a section where cudaMalloc's implicit device-wide
 * synchronisation is not acceptable).  It has no counterpart in the reference,
 * which runs on the CPU and allocates its scratch with aligned_alloc on every
 * call.  This entry point calls no cudaMalloc / cudaFree and needs no sdq_init
 * and no weight handle: the weight is given as device pointers (int8 [N,K] and
 * fp32 [N]) and the int8 activations and row scales live in a fixed array that is
 * part of the library image, held on every GPU that loads the library until the
 * process exits (about 32.1 MiB).  Limits: M <= SDQ_STATIC_MAX_ROWS and
 * M*K <= SDQ_STATIC_MAX_AQ_BYTES, else SDQ_ERR_INVALID.  All calls on a device
 * share that array: calls that can overlap on the GPU race; order them (one
 * stream, or events).  A, out and bias are device memory (SDQ_A_HOST /
 * SDQ_OUT_HOST are rejected: staging would need an allocation).  The first call
 * on each device does a one-time host-side set-up; make it before any stream
 * capture begins.  A bounded wait that gives up inside the GEMM kernel leaves a
 * code in the array; only a call made with SDQ_SYNC reads it (after waiting for
 * the stream) and returns SDQ_ERR_DEVICE_TIMEOUT -- for its own kernels or for
 * those of earlier calls -- so a caller that never passes SDQ_SYNC is never
 * told.  The pointers w_scale_dev and bias_dev may have any 4-byte alignment. */
#define SDQ_STATIC_MAX_ROWS 32768
#define SDQ_STATIC_MAX_AQ_BYTES 33554432
SDQ_API int sdq_qgemm_static_scratch(const int8_t* wq_dev, const float* w_scale_dev, int64_t N,
                                     int64_t K, const float* A_dev, int64_t M, float* out_dev,
                                     const float* bias_dev, uint32_t flags, void* stream);

/* ---- weight quantizers ---- */

/* Quantizes `rows` rows of `last` elements to int8 with one fp32 scale per row.
 * SDQ_MODE_PACKER is byte-identical to quant_rows of the .sdcpp packer
 * (tools/quantize/pack_sdcpp.py:38-51: x*(127/amax), round half even, clip,
 * scale amax/127 and 0 for an all-zero row); SDQ_MODE_ROWWISE to
 * sd::quantize_rowwise (src/core/tensor.h:55, src/core/tensor.cpp:63-78:
 * x/(amax/127), round half away, scale 1 for an all-zero row; fp32 source only). */
SDQ_API int sdq_quantize_rows(const void* src, int src_dtype, int64_t rows, int64_t last, int mode,
                      int8_t* q, float* scale, uint32_t flags, void* stream);

/* w[r,c] = q[r,c] * scale[r] -- replaces dequant_pack (src/model/ovi_dit.cpp:53-63). */
SDQ_API int sdq_dequant_rows(const int8_t* q, const float* scale, int64_t rows, int64_t last, float* w,
                     uint32_t flags, void* stream);

/* ---- .sdcpp packs ---- */

/* Offline packer -- replaces tools/quantize/pack_sdcpp.py main() (lines 54-124):
 * reads a .safetensors file, quantizes every float tensor with numel >= 65536
 * that is not excluded (row = last dim) on the GPU, keeps the rest as raw fp32,
 * and writes a .sdcpp v1 file that is byte-identical to the python packer's.
 * `only`: comma-separated name prefixes ("" = all); `dtype_preserve`:
 * colon-separated source dtypes kept raw ("" = none). */
SDQ_API int sdq_pack_sdcpp(const char* safetensors_in, const char* sdcpp_out, const char* only,
                   const char* dtype_preserve);

typedef struct sdq_pack sdq_pack; /* an open .sdcpp file */

#define SDQ_DT_F32 0 /* codes of sdq_entry.dtype: sd::DType values (src/core/tensor.h:13) */
#define SDQ_DT_I8 2

typedef struct sdq_entry {
  const char* name;    /* NUL-terminated, owned by the pack */
  int32_t dtype;       /* SDQ_DT_I8 or SDQ_DT_F32 */
  int32_t ndim;
  int64_t dims[8];
  const void* data;    /* view into the file mapping (host) */
  uint64_t nbytes;
  uint64_t file_offset; /* of `data` from the start of the file */
  sdq_weight_t weight; /* device copy of an I8 entry when the pack was opened with
                          SDQ_PACK_UPLOAD, viewed as [numel/last, last]; else 0 */
  uint64_t name_len;   /* bytes of `name` (a name may contain NUL bytes; the file stores a length) */
} sdq_entry;

#define SDQ_PACK_UPLOAD 0x1u /* upload every I8 entry (+ scales) to the device at open */

/* Opens and validates a .sdcpp v1 file -- replaces sd::load_sdcpp
 * (src/serde/sdcpp.h:18-19, src/serde/sdcpp.cpp:47-133).  Entries appear as the
 * reference's map does: a quantized tensor as `name` (I8, original shape) plus
 * `name.scale` (F32 [rows]), a raw tensor as `name` (F32).  Failures carry the
 * reference's messages ("sdcpp: bad magic", "sdcpp: truncated file", ...). */
SDQ_API int sdq_pack_open(const char* path, uint32_t flags, sdq_pack** out);
SDQ_API int64_t sdq_pack_count(const sdq_pack* p);
/* 1 when the file mapping could be page-locked at open (uploads were direct DMA), else 0. */
SDQ_API int sdq_pack_pinned(const sdq_pack* p);
SDQ_API int sdq_pack_entry(const sdq_pack* p, int64_t index, sdq_entry* out);
SDQ_API int sdq_pack_find(const sdq_pack* p, const char* name, sdq_entry* out);
/* Unmaps the file and releases the device copies made at open. */
SDQ_API int sdq_pack_close(sdq_pack* p);

#ifdef __cplusplus
}
#endif
#endif /* SDQ_H */
