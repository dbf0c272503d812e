// C wrappers around the UNMODIFIED reference implementation of the int8
// quantized-linear path (sd::qgemm, sd::quantize_rowwise, sd::load_sdcpp),
// compiled from the reference's own source files where they lie -- see the
// Makefile beside this file.  TEST INFRASTRUCTURE ONLY: it validates the C
// restatement in qgemm_oracle.c and serves as the timed CPU baseline.  The
// reference's sources are never copied; this file only calls their public API
// (src/core/tensor.h:48-61, src/serde/sdcpp.h:18-19).
#include "core/tensor.h"
#include "serde/sdcpp.h"
#include "model/blocks.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <exception>
#include <map>
#include <string>

namespace {
sd::Tensor view(const void* p, std::vector<int64_t> shape, sd::DType dt, size_t nbytes) {
  sd::Tensor t;
  t.shape = std::move(shape);
  t.dtype = dt;
  t.data = const_cast<void*>(p);
  t.nbytes = nbytes;
  t.owning = false;
  return t;
}
}  // namespace

extern "C" {

int sdref_nthreads() { return sd::nthreads(); }
void sdref_set_nthreads(int n) { sd::set_nthreads(n); }

// out must hold M*N floats.  Returns the number of floats written.
int64_t sdref_qgemm(const float* A, int64_t M, int64_t K, const int8_t* Bq, int64_t N,
                    const float* bs, float* out) {
  sd::Tensor a = view(A, {M, K}, sd::DType::F32, (size_t)M * K * 4);
  sd::Tensor b = view(Bq, {N, K}, sd::DType::I8, (size_t)N * K);
  sd::Tensor s = view(bs, {N}, sd::DType::F32, (size_t)N * 4);
  sd::Tensor o;
  sd::qgemm(a, b, s, o);
  if (o.data && o.nbytes) std::memcpy(out, o.data, o.nbytes);
  return (int64_t)(o.nbytes / 4);
}

// Timed variant for the benchmark: runs qgemm `reps` times and returns the best
// wall time in seconds; the result of the last run is discarded.
double sdref_qgemm_time(const float* A, int64_t M, int64_t K, const int8_t* Bq, int64_t N,
                        const float* bs, int reps);

void sdref_quantize_rowwise(const float* W, int64_t N, int64_t K, int8_t* q, float* scale) {
  sd::Tensor w = view(W, {N, K}, sd::DType::F32, (size_t)N * K * 4);
  sd::Tensor wq, sc;
  sd::quantize_rowwise(w, wq, sc);
  std::memcpy(q, wq.data, wq.nbytes);
  std::memcpy(scale, sc.data, sc.nbytes);
}

// blk::layernorm without affine parameters (src/model/blocks.cpp:18-43), as ffn_fwd and
// block_self_fwd call it (src/model/ovi_dit.cpp:205-217).
void sdref_layernorm(const float* x, int64_t M, int64_t K, float eps, float* y) {
  sd::Tensor t = view(x, {M, K}, sd::DType::F32, (size_t)M * K * 4);
  sd::Tensor o;
  sd::blk::layernorm(t, o, nullptr, nullptr, eps);
  std::memcpy(y, o.data, o.nbytes);
}

// blk::layernorm with its affine parameters (weight, bias: fp32 [K]), as block_vanilla_fwd and
// fusion_cross_ffn call it in front of the cross-attention projections
// (src/model/ovi_dit.cpp:241, :264).
void sdref_layernorm_affine(const float* x, int64_t M, int64_t K, const float* w, const float* b,
                            float eps, float* y) {
  sd::Tensor t = view(x, {M, K}, sd::DType::F32, (size_t)M * K * 4);
  sd::Tensor wt = view(w, {K}, sd::DType::F32, (size_t)K * 4);
  sd::Tensor bt = view(b, {K}, sd::DType::F32, (size_t)K * 4);
  sd::Tensor o;
  sd::blk::layernorm(t, o, &wt, &bt, eps);
  std::memcpy(y, o.data, o.nbytes);
}

// sd::matmul (src/core/tensor.h:46, src/core/gemm.cpp:115-160): out[M,N] = a[M,K] * w[K,N] + bias.
void sdref_matmul(const float* a, int64_t M, int64_t K, const float* w, int64_t N,
                  const float* bias_or_null, float* out) {
  sd::Tensor at = view(a, {M, K}, sd::DType::F32, (size_t)M * K * 4);
  sd::Tensor wt = view(w, {K, N}, sd::DType::F32, (size_t)K * N * 4);
  sd::Tensor o;
  sd::matmul(at, wt, o, bias_or_null);
  if (o.data && o.nbytes) std::memcpy(out, o.data, o.nbytes);
}

// blk::sdpa (src/model/blocks.h:60-66, src/model/blocks.cpp:113-199): out[Lq,C] =
// softmax(q k^T / sqrt(hd)) v per head, exact fp32, no causal mask.
void sdref_sdpa(const float* q, const float* k, const float* v, int64_t Lq, int64_t Lk, int64_t C,
                int heads, float* out) {
  sd::Tensor qt = view(q, {Lq, C}, sd::DType::F32, (size_t)Lq * C * 4);
  sd::Tensor kt = view(k, {Lk, C}, sd::DType::F32, (size_t)Lk * C * 4);
  sd::Tensor vt = view(v, {Lk, C}, sd::DType::F32, (size_t)Lk * C * 4);
  sd::Tensor o;
  sd::blk::sdpa(qt, kt, vt, heads, o, false);
  if (o.data && o.nbytes) std::memcpy(out, o.data, o.nbytes);
}

void sdref_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  sd::Tensor s = view(src, {n}, sd::DType::F32, (size_t)n * 4);
  sd::Tensor o;
  sd::to_bf16(s, o);
  std::memcpy(dst, o.data, o.nbytes);
}

// Loads `path` with the reference loader and writes a listing, one line per
// entry sorted by name: "name dtype ndim d0,d1,.. offset nbytes" where offset is
// the view's byte offset from the start of the file mapping.  Returns the
// number of entries, or -1 with the exception text in `buf` when it throws.
int64_t sdref_load_sdcpp_listing(const char* path, char* buf, int64_t buflen) {
  try {
    std::shared_ptr<void> owner;
    auto m = sd::load_sdcpp(path, owner);
    std::map<std::string, const sd::Tensor*> sorted;
    for (auto& kv : m) sorted[kv.first] = &kv.second;
    std::string s;
    for (auto& kv : sorted) {
      const sd::Tensor& t = *kv.second;
      s += kv.first + " " + std::to_string((int)t.dtype) + " " + std::to_string(t.shape.size()) + " ";
      for (size_t i = 0; i < t.shape.size(); i++)
        s += (i ? "," : "") + std::to_string(t.shape[i]);
      if (t.shape.empty()) s += "-";
      s += " " + std::to_string((const char*)t.data - (const char*)owner.get()) + " " +
           std::to_string(t.nbytes) + "\n";
    }
    if ((int64_t)s.size() + 1 > buflen) { std::snprintf(buf, buflen, "listing too long"); return -2; }
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return (int64_t)m.size();
  } catch (const std::exception& e) {
    std::snprintf(buf, buflen, "%s", e.what());
    return -1;
  }
}

}  // extern "C"

#include <chrono>
extern "C" double sdref_qgemm_time(const float* A, int64_t M, int64_t K, const int8_t* Bq,
                                   int64_t N, const float* bs, int reps) {
  sd::Tensor a = view(A, {M, K}, sd::DType::F32, (size_t)M * K * 4);
  sd::Tensor b = view(Bq, {N, K}, sd::DType::I8, (size_t)N * K);
  sd::Tensor s = view(bs, {N}, sd::DType::F32, (size_t)N * 4);
  double best = 1e30;
  for (int r = 0; r < std::max(1, reps); r++) {
    sd::Tensor o;
    auto t0 = std::chrono::steady_clock::now();
    sd::qgemm(a, b, s, o);
    double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    best = std::min(best, dt);
  }
  return best;
}
