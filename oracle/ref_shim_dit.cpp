// C wrappers around the UNMODIFIED caller side of the reference's int8 linear: the helper
// functions that sit either side of sd::qgemm in src/model/ovi_dit.cpp (mlin :66-84,
// gelu_tanh_inplace :132-142, gated_add_inplace :152-159, mod_rows :162-173, ffn_fwd :214-222).
// They live in an anonymous namespace of that file, so this translation unit includes the file
// where it lies (the include path comes from the Makefile beside this file) and adds wrappers
// inside the same namespace.  TEST INFRASTRUCTURE ONLY; nothing of the reference is copied.
#include "model/ovi_dit.cpp"

#include <cstring>
#include <vector>

namespace sd {
namespace ovi {
namespace {

Tensor dit_view(const void* p, std::vector<int64_t> shape, DType dt, size_t nbytes) {
  Tensor t;
  t.shape = std::move(shape);
  t.dtype = dt;
  t.data = const_cast<void*>(p);
  t.nbytes = nbytes;
  t.owning = false;
  return t;
}

// An int8 Linear as load_quantized_pack builds it: int8 [N,K] view with the fp32 row scales
// directly behind the bytes (mlin finds them with scale_after), optional fp32 bias view.
struct PackedLinear {
  std::vector<char> blob;
  blk::Linear lin;
  PackedLinear(const int8_t* q, const float* s, const float* bias, int64_t N, int64_t K)
      : blob((size_t)N * K + (size_t)N * 4) {
    std::memcpy(blob.data(), q, (size_t)N * K);
    std::memcpy(blob.data() + (size_t)N * K, s, (size_t)N * 4);
    lin.w = dit_view(blob.data(), {N, K}, DType::I8, (size_t)N * K);
    if (bias) lin.b = dit_view(bias, {N}, DType::F32, (size_t)N * 4);
  }
};

}  // namespace
}  // namespace ovi
}  // namespace sd

using namespace sd;
using namespace sd::ovi;

extern "C" {

// x[L,C] += y[L,C] * gate[C], in place on x.
void sdref_gated_add(float* x, const float* y, const float* gate, int64_t L, int64_t C) {
  Tensor xt = dit_view(x, {L, C}, DType::F32, (size_t)L * C * 4);
  gated_add_inplace(xt, dit_view(y, {L, C}, DType::F32, (size_t)L * C * 4),
                    dit_view(gate, {C}, DType::F32, (size_t)C * 4));
}

void sdref_add(float* x, const float* y, int64_t n) {
  Tensor xt = dit_view(x, {n}, DType::F32, (size_t)n * 4);
  add_inplace(xt, dit_view(y, {n}, DType::F32, (size_t)n * 4));
}

void sdref_mod_rows(const float* x, const float* shift, const float* scale, int64_t L, int64_t C,
                    float* y) {
  Tensor o;
  mod_rows(dit_view(x, {L, C}, DType::F32, (size_t)L * C * 4),
           dit_view(shift, {C}, DType::F32, (size_t)C * 4),
           dit_view(scale, {C}, DType::F32, (size_t)C * 4), o);
  std::memcpy(y, o.data, o.nbytes);
}

void sdref_gelu_tanh(float* x, int64_t n) {
  Tensor xt = dit_view(x, {n}, DType::F32, (size_t)n * 4);
  gelu_tanh_inplace(xt);
}

// mlin on an int8 weight: qgemm + the separate bias pass.  y holds M*N floats.
void sdref_mlin_i8(const float* x, int64_t M, int64_t K, const int8_t* q, const float* s,
                   const float* bias_or_null, int64_t N, float* y) {
  PackedLinear l(q, s, bias_or_null, N, K);
  Tensor o;
  mlin(dit_view(x, {M, K}, DType::F32, (size_t)M * K * 4), l.lin, o);
  std::memcpy(y, o.data, o.nbytes);
}

// The whole ffn_fwd: x[M,D] is updated in place; e is the [6,D] modulation table whose rows
// 3, 4, 5 are the FFN's shift, scale and gate.
void sdref_ffn_fwd(float* x, int64_t M, int64_t D, int64_t F, const float* e, const int8_t* q1,
                   const float* s1, const float* b1, const int8_t* q2, const float* s2,
                   const float* b2) {
  PackedLinear l1(q1, s1, b1, F, D), l2(q2, s2, b2, D, F);
  BlockW b;
  b.ffn.fc1.w = dit_view(l1.lin.w.data, {F, D}, DType::I8, (size_t)F * D);
  b.ffn.fc2.w = dit_view(l2.lin.w.data, {D, F}, DType::I8, (size_t)D * F);
  if (b1) b.ffn.fc1.b = dit_view(b1, {F}, DType::F32, (size_t)F * 4);
  if (b2) b.ffn.fc2.b = dit_view(b2, {D}, DType::F32, (size_t)D * 4);
  Tensor xt = dit_view(x, {M, D}, DType::F32, (size_t)M * D * 4);
  ffn_fwd(b, xt, dit_view(e, {6, D}, DType::F32, (size_t)6 * D * 4));
}

}  // extern "C"
