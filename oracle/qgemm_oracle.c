/*
 * CPU oracle for the int8 quantized-linear path -- TEST INFRASTRUCTURE ONLY.
 * See qgemm_oracle.h.  Built with -ffp-contract=off so that no multiply-add is
 * fused: every fp32 operation below is one IEEE-754 round-to-nearest-even
 * operation, which is what the reference's expressions on this path compile to
 * (they contain no a*b+c pattern except GELU, which is tolerance-checked).
 *
 * Citations are into JasonHonKL/Self-evolve-diffusion-cpp.
 */
#include "qgemm_oracle.h"

#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

/* ---- a minimal fork-join helper: rows [0,n) in contiguous slices ---- */
static int g_threads = 0;

void orc_set_threads(int n) { g_threads = n > 0 ? n : 0; }

int orc_threads(void) {
  if (g_threads > 0) return g_threads;
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

typedef void (*range_fn)(int64_t begin, int64_t end, void* ctx);
typedef struct { range_fn fn; void* ctx; int64_t b, e; } slice_t;

static void* slice_main(void* p) {
  slice_t* s = (slice_t*)p;
  s->fn(s->b, s->e, s->ctx);
  return NULL;
}

static void par_rows(int64_t n, range_fn fn, void* ctx) {
  int nt = orc_threads();
  if (nt > 256) nt = 256;
  if ((int64_t)nt > n) nt = (int)n;
  if (nt <= 1) { if (n > 0) fn(0, n, ctx); return; }
  pthread_t th[256];
  slice_t sl[256];
  int started = 0;
  for (int t = 0; t < nt; t++) {
    sl[t].fn = fn; sl[t].ctx = ctx;
    sl[t].b = n * t / nt; sl[t].e = n * (t + 1) / nt;
    if (t == nt - 1 || pthread_create(&th[t], NULL, slice_main, &sl[t]) != 0) {
      sl[t].e = n; /* run the remainder on this thread */
      slice_main(&sl[t]);
      break;
    }
    started++;
  }
  for (int t = 0; t < started; t++) pthread_join(th[t], NULL);
}

/* src/core/tensor.cpp:39-43: add 0x7fff + lsb, keep the high half. */
void orc_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    uint32_t u;
    memcpy(&u, &src[i], 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    dst[i] = (uint16_t)(u >> 16);
  }
}

/* src/core/tensor.cpp:44-47 and tools/quantize/pack_sdcpp.py:40-41. */
void orc_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    uint32_t u = (uint32_t)src[i] << 16;
    memcpy(&dst[i], &u, 4);
  }
}

/* tools/quantize/pack_sdcpp.py:42: numpy's exact binary16 -> binary32 widening. */
void orc_f16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    uint32_t h = src[i], sign = (h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu, u;
    if (e == 0) {
      if (m == 0) {
        u = sign;
      } else { /* subnormal half: renormalise */
        int sh = 0;
        while (!(m & 0x400u)) { m <<= 1; sh++; }
        m &= 0x3ffu;
        u = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | (m << 13);
      }
    } else if (e == 31) {
      u = sign | 0x7f800000u | (m << 13);
    } else {
      u = sign | ((e + 127 - 15) << 23) | (m << 13);
    }
    memcpy(&dst[i], &u, 4);
  }
}

/* src/core/qgemm.cpp:62-69.  The reference converts with the SSE instruction
 * cvtss2si: round to nearest even under the default mode, and the "integer
 * indefinite" INT_MIN for NaN or a magnitude that does not fit 32 bits.  Then
 * it clamps to [-127,127]. */
static int round_clamp_i8(float x) {
  int v;
  if (!(fabsf(x) < 2147483648.0f)) v = INT_MIN; /* NaN, inf, out of range */
  else v = (int)lrintf(x);                      /* default mode = RNE */
  if (v > 127) v = 127;
  if (v < -127) v = -127;
  return v;
}

/* ---- per-range bodies; the exported functions below fan them out ---- */
typedef struct {
  const float* A; const int8_t* aq_in; const int8_t* bq; const int32_t* acc_in;
  const float* as_in; const float* bs; const float* bias;
  int8_t* aq; float* as; int32_t* acc; float* out;
  int64_t M, N, K;
} job_t;

/* src/core/qgemm.cpp:84-96. */
static void act_quant_range(int64_t b, int64_t e, void* p) {
  job_t* j = (job_t*)p;
  const int64_t K = j->K;
  for (int64_t i = b; i < e; i++) {
    const float* r = j->A + i * K;
    float mx = 0.0f;
    for (int64_t k = 0; k < K; k++) {
      float f = fabsf(r[k]);
      mx = (mx < f) ? f : mx; /* std::max(mx, f): a NaN f is ignored */
    }
    float sc = mx / 127.0f;
    if (sc == 0.0f) sc = 1.0f;
    j->as[i] = sc;
    const float inv = 1.0f / sc;
    int8_t* q = j->aq + i * K;
    for (int64_t k = 0; k < K; k++) q[k] = (int8_t)round_clamp_i8(r[k] * inv);
  }
}

void orc_act_quant_rows(const float* A, int64_t M, int64_t K, int8_t* aq, float* as) {
  job_t j = {0};
  j.A = A; j.aq = aq; j.as = as; j.M = M; j.K = K;
  par_rows(M, act_quant_range, &j);
}

/* src/core/qgemm.cpp:22-59: plain s32 sums; integer addition is exact and
 * order-free, so the AVX2 lanes, the s16-widened branch (M >= 2048) and the
 * scalar tail all produce this value.  Ranges are over groups of 16 weight
 * rows so that a group's bytes stay in cache across the M loop. */
static void dot_range(int64_t gb, int64_t ge, void* p) {
  job_t* jb = (job_t*)p;
  const int64_t M = jb->M, N = jb->N, K = jb->K;
  for (int64_t g = gb; g < ge; g++) {
    int64_t j0 = g * 16, j1 = j0 + 16 < N ? j0 + 16 : N;
    for (int64_t i = 0; i < M; i++) {
      const int8_t* a = jb->aq_in + i * K;
      for (int64_t j = j0; j < j1; j++) {
        const int8_t* b = jb->bq + j * K;
        int32_t s = 0;
        for (int64_t k = 0; k < K; k++) s += (int32_t)a[k] * (int32_t)b[k];
        jb->acc[i * N + j] = s;
      }
    }
  }
}

void orc_dot_s32(const int8_t* aq, const int8_t* bq, int64_t M, int64_t N, int64_t K,
                 int32_t* acc) {
  job_t j = {0};
  j.aq_in = aq; j.bq = bq; j.acc = acc; j.M = M; j.N = N; j.K = K;
  par_rows((N + 15) / 16, dot_range, &j);
}

/* src/core/qgemm.cpp:123-124,135: the two scales are multiplied first. */
static void rescale_range(int64_t b, int64_t e, void* p) {
  job_t* j = (job_t*)p;
  const int64_t N = j->N;
  for (int64_t i = b; i < e; i++)
    for (int64_t c = 0; c < N; c++)
      j->out[i * N + c] = (float)j->acc_in[i * N + c] * (j->as_in[i] * j->bs[c]);
}

void orc_rescale(const int32_t* acc, const float* as, const float* bs, int64_t M, int64_t N,
                 float* out) {
  job_t j = {0};
  j.acc_in = acc; j.as_in = as; j.bs = bs; j.out = out; j.M = M; j.N = N;
  par_rows(M, rescale_range, &j);
}

/* src/core/qgemm.cpp:73-142. */
void orc_qgemm(const float* A, const int8_t* Bq, const float* bs, int64_t M, int64_t N,
               int64_t K, float* out) {
  if (M == 0 || N == 0) return;
  if (K == 0) { /* the reference returns its zero-initialised tensor (:75-76) */
    memset(out, 0, (size_t)M * (size_t)N * 4);
    return;
  }
  int8_t* aq = (int8_t*)malloc((size_t)M * (size_t)K);
  float* as = (float*)malloc((size_t)M * 4);
  int32_t* acc = (int32_t*)malloc((size_t)M * (size_t)N * 4);
  orc_act_quant_rows(A, M, K, aq, as);
  orc_dot_s32(aq, Bq, M, N, K, acc);
  orc_rescale(acc, as, bs, M, N, out);
  free(acc);
  free(as);
  free(aq);
}

/* src/model/ovi_dit.cpp:71-79. */
static void bias_range(int64_t b, int64_t e, void* p) {
  job_t* j = (job_t*)p;
  const int64_t N = j->N;
  for (int64_t i = b; i < e; i++)
    for (int64_t c = 0; c < N; c++) j->out[i * N + c] += j->bias[c];
}

void orc_bias_add(float* y, const float* b, int64_t M, int64_t N) {
  job_t j = {0};
  j.out = y; j.bias = b; j.M = M; j.N = N;
  par_rows(M, bias_range, &j);
}

/* x += y * gate (src/model/ovi_dit.cpp:152-159) or x += y (src/model/ovi_dit.cpp:144-149).
 * The reference is built -O3 for an FMA target, where GCC contracts x + y*g into one fused
 * multiply-add; fmaf states that explicitly (this file is built with contraction off) and is
 * bit-identical to the compiled reference function. */
static void residual_range(int64_t b, int64_t e, void* p) {
  job_t* j = (job_t*)p;
  const int64_t N = j->N;
  const float* y = j->A;
  const float* gate = j->bias;
  for (int64_t i = b; i < e; i++)
    for (int64_t c = 0; c < N; c++)
      j->out[i * N + c] = gate ? fmaf(y[i * N + c], gate[c], j->out[i * N + c])
                               : j->out[i * N + c] + y[i * N + c];
}

void orc_residual_add(float* x, const float* y, const float* gate_or_null, int64_t M, int64_t N) {
  job_t j = {0};
  j.out = x; j.A = y; j.bias = gate_or_null; j.M = M; j.N = N;
  par_rows(M, residual_range, &j);
}

/* src/model/ovi_dit.cpp:132-142.  tanhf differs between libms by an ulp or
 * two, so this one is compared under a tolerance, never bit-for-bit. */
static void gelu_range(int64_t b, int64_t e, void* p) {
  float* x = ((job_t*)p)->out;
  for (int64_t i = b; i < e; i++) {
    float v = x[i];
    float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    x[i] = 0.5f * v * (1.0f + tanhf(u));
  }
}

void orc_gelu_tanh(float* x, int64_t n) {
  job_t j = {0};
  j.out = x;
  par_rows(n, gelu_range, &j);
}

/* src/core/tensor.cpp:63-78: divide by the scale, round half AWAY from zero
 * (std::lround), no clamp, scale 1 for an all-zero row. */
static void rowwise_range(int64_t b, int64_t e, void* p) {
  job_t* j = (job_t*)p;
  const int64_t K = j->K;
  const float* W = j->A;
  for (int64_t i = b; i < e; i++) {
    float mx = 0.0f;
    for (int64_t k = 0; k < K; k++) {
      float f = fabsf(W[i * K + k]);
      mx = (mx < f) ? f : mx;
    }
    float sc = mx / 127.0f;
    if (sc == 0.0f) sc = 1.0f;
    j->as[i] = sc;
    for (int64_t k = 0; k < K; k++) j->aq[i * K + k] = (int8_t)lroundf(W[i * K + k] / sc);
  }
}

void orc_quantize_rowwise(const float* W, int64_t N, int64_t K, int8_t* q, float* scale) {
  job_t j = {0};
  j.A = W; j.aq = q; j.as = scale; j.K = K;
  par_rows(N, rowwise_range, &j);
}

/* tools/quantize/pack_sdcpp.py:45-51 under numpy 2.x promotion rules: every
 * array stays float32, so  inv = 127f / (amax > 0 ? amax : 1f)  is one fp32
 * division, x*inv one fp32 multiply, np.rint rounds half to EVEN, the clip is
 * to [-127,127], and the stored scale is the fp32 division amax / 127f (0 for
 * an all-zero row).  np.max propagates NaN; such rows are outside the contract. */
static void packer_range(int64_t b, int64_t e, void* p) {
  job_t* j = (job_t*)p;
  const int64_t last = j->K;
  for (int64_t i = b; i < e; i++) {
    const float* r = j->A + i * last;
    float amax = 0.0f;
    for (int64_t k = 0; k < last; k++) {
      float f = fabsf(r[k]);
      if (f > amax) amax = f;
    }
    const float safe = amax > 0.0f ? amax : 1.0f;
    const float inv = 127.0f / safe;
    for (int64_t k = 0; k < last; k++) {
      float v = nearbyintf(r[k] * inv);
      if (v > 127.0f) v = 127.0f;
      if (v < -127.0f) v = -127.0f;
      j->aq[i * last + k] = (int8_t)v;
    }
    j->as[i] = amax / 127.0f;
  }
}

void orc_quant_rows_packer(const float* x, int64_t rows, int64_t last, int8_t* q, float* scale) {
  job_t j = {0};
  j.A = x; j.aq = q; j.as = scale; j.K = last;
  par_rows(rows, packer_range, &j);
}

/* sd::matmul, the portable branch (src/core/gemm.cpp:100-110): out[i,j] = sum_k a[i,k]*w[k,j]
 * added left to right in fp32, then the separate bias pass (src/core/gemm.cpp:33-40).  The
 * reference's AVX2 / BLAS branches add in other orders, so every comparison with this function
 * is under the reference's own matmul tolerance, never bit for bit. */
typedef struct { const float* a; const float* w; const float* bias; float* out; int64_t N, K; } mm_t;
static void mm_range(int64_t b, int64_t e, void* p) {
  mm_t* j = (mm_t*)p;
  for (int64_t i = b; i < e; i++)
    for (int64_t c = 0; c < j->N; c++) {
      float s = 0.0f;
      for (int64_t k = 0; k < j->K; k++) s += j->a[i * j->K + k] * j->w[k * j->N + c];
      j->out[i * j->N + c] = j->bias ? s + j->bias[c] : s;
    }
}
void orc_matmul_f32(const float* a, int64_t M, int64_t K, const float* w, int64_t N,
                    const float* bias_or_null, float* out) {
  mm_t j = {a, w, bias_or_null, out, N, K};
  par_rows(M, mm_range, &j);
}

/* blk::sdpa, the portable branch (src/model/blocks.cpp:146-152, 156-166, 183-190): per head and
 * query row, scores s_j = (sum_d q_d k_jd) * scale added left to right, mx = max s_j,
 * s_j = exp(s_j - mx), sum, s_j *= 1/sum, then o_d = sum_j s_j * v_jd.  (That branch multiplies
 * the already normalised s_j by inv once more -- a slip the AVX2 branch the reference is built
 * with does not have; the restatement follows the AVX2 branch's arithmetic: normalise once.)
 * expf and the summation orders differ between builds, so comparisons are under a tolerance. */
typedef struct { const float* q; const float* k; const float* v; float* out; int64_t Lq, Lk, C; int heads; } sdpa_t;
static void sdpa_range(int64_t b, int64_t e, void* p) {
  sdpa_t* j = (sdpa_t*)p;
  const int64_t hd = j->C / j->heads;
  const float scale = 1.0f / sqrtf((float)hd);
  float* s = (float*)malloc((size_t)(j->Lk > 0 ? j->Lk : 1) * sizeof(float));
  for (int64_t it = b; it < e; it++) {
    const int64_t h = it / j->Lq, i = it % j->Lq;
    const float* qi = j->q + i * j->C + h * hd;
    float mx = -INFINITY;
    for (int64_t t = 0; t < j->Lk; t++) {
      const float* kt = j->k + t * j->C + h * hd;
      float d = 0.0f;
      for (int64_t c = 0; c < hd; c++) d += qi[c] * kt[c];
      s[t] = d * scale;
      if (s[t] > mx) mx = s[t];
    }
    float sum = 0.0f;
    for (int64_t t = 0; t < j->Lk; t++) { s[t] = expf(s[t] - mx); sum += s[t]; }
    const float inv = 1.0f / sum;
    float* o = j->out + i * j->C + h * hd;
    for (int64_t c = 0; c < hd; c++) o[c] = 0.0f;
    for (int64_t t = 0; t < j->Lk; t++) {
      const float w = s[t] * inv;
      const float* vt = j->v + t * j->C + h * hd;
      for (int64_t c = 0; c < hd; c++) o[c] += w * vt[c];
    }
  }
  free(s);
}
void orc_sdpa(const float* q, const float* k, const float* v, int64_t Lq, int64_t Lk, int64_t C,
              int heads, float* out) {
  sdpa_t j = {q, k, v, out, Lq, Lk, C, heads};
  par_rows(Lq * heads, sdpa_range, &j);
}

/* src/model/ovi_dit.cpp:53-63. */
void orc_dequant_rows(const int8_t* q, const float* scale, int64_t rows, int64_t last, float* w) {
  for (int64_t i = 0; i < rows; i++)
    for (int64_t k = 0; k < last; k++) w[i * last + k] = (float)q[i * last + k] * scale[i];
}

/* src/model/blocks.cpp:18-43 (w = b = null) then src/model/ovi_dit.cpp:162-173. */
typedef struct { const float* x; const float* shift; const float* scale; float* y; int64_t K; float eps; int affine; } ln_t;

static void ln_range(int64_t b, int64_t e, void* p) {
  ln_t* j = (ln_t*)p;
  const int64_t N = j->K;
  for (int64_t i = b; i < e; i++) {
    const float* r = j->x + i * N;
    float mu = 0.0f;
    for (int64_t k = 0; k < N; k++) mu += r[k];
    mu /= (float)N;
    float var = 0.0f;
    for (int64_t k = 0; k < N; k++) {
      float d = r[k] - mu;
      var += d * d;
    }
    const float inv = 1.0f / sqrtf(var / (float)N + j->eps);
    float* o = j->y + i * N;
    for (int64_t k = 0; k < N; k++) {
      if (j->affine) {
        /* blk::layernorm with weight and bias (src/model/blocks.cpp:39-40): the reference's
         * build fuses the last multiply and the add, as checked against the compiled function */
        o[k] = fmaf((r[k] - mu) * inv, j->scale[k], j->shift[k]);
        continue;
      }
      const float ln = (r[k] - mu) * inv * 1.0f + 0.0f;
      /* mod_rows (src/model/ovi_dit.cpp:162-173): one fused multiply-add in the reference's
       * -O3 build for an FMA target, as checked against the compiled function */
      o[k] = fmaf(ln, 1.0f + j->scale[k], j->shift[k]);
    }
  }
}

void orc_layernorm_mod(const float* x, int64_t M, int64_t K, const float* shift,
                       const float* scale, float eps, float* y) {
  ln_t j = {x, shift, scale, y, K, eps, 0};
  par_rows(M, ln_range, &j);
}

void orc_layernorm_affine(const float* x, int64_t M, int64_t K, const float* weight,
                          const float* bias, float eps, float* y) {
  ln_t j = {x, bias, weight, y, K, eps, 1};
  par_rows(M, ln_range, &j);
}
