// Standalone test of libsd_b200.so, written the way the reference's own tests are
// (tests/test_core.cpp, tests/test_sdcpp.cpp: a main(), CHECK macros, cosine gates)
// but against the B200 drop-in.  `test_dropin --cpu <golden_dir>` runs only what
// needs no GPU (containers, loader format errors, thread dispatch);
// `test_dropin <golden_dir>` runs everything.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "core/tensor.h"
#include "model/blocks.h"
#include "serde/sdcpp.h"

using namespace sd;

static int g_fail = 0;
#define CHECK(cond)                                                       \
  do {                                                                    \
    if (!(cond)) {                                                        \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);         \
      g_fail++;                                                           \
    }                                                                     \
  } while (0)

static void fill_uniform(Tensor& t, uint64_t seed) {  // xorshift in [-1,1)
  float* p = t.ptr<float>();
  uint64_t s = seed ? seed : 0x9e3779b97f4a7c15ull;
  for (int64_t i = 0, n = t.numel(); i < n; i++) {
    s ^= s << 13; s ^= s >> 7; s ^= s << 17;
    p[i] = ((int32_t)(s >> 40) % 20001 - 10000) / 10000.f;
  }
}

static double cosine(const float* a, const float* b, int64_t n) {
  double ab = 0, aa = 0, bb = 0;
  for (int64_t i = 0; i < n; i++) { ab += (double)a[i] * b[i]; aa += (double)a[i] * a[i]; bb += (double)b[i] * b[i]; }
  return ab / (std::sqrt(aa) * std::sqrt(bb) + 1e-30);
}

static bool throws(const std::string& path, std::string* what = nullptr) {
  try {
    std::shared_ptr<void> owner;
    load_sdcpp(path, owner);
  } catch (const std::runtime_error& e) {
    if (what) *what = e.what();
    return true;
  }
  return false;
}

static void test_containers() {
  Tensor t({3, 5}, DType::F32);
  CHECK(t.numel() == 15 && t.rows() == 3 && t.cols() == 5 && t.nbytes == 60 && t.owning);
  CHECK(((uintptr_t)t.data & 63) == 0);
  for (int i = 0; i < 15; i++) CHECK(t.ptr<float>()[i] == 0.f);
  Tensor u = std::move(t);
  CHECK(t.data == nullptr && u.numel() == 15);
  u.reshape({5, 3});
  CHECK(u.rows() == 5);
  Tensor x({1000}, DType::F32), b, back;
  fill_uniform(x, 7);
  to_bf16(x, b);
  to_f32(b, back);
  CHECK(b.dtype == DType::BF16 && b.nbytes == 2000);
  for (int i = 0; i < 1000; i++) CHECK(std::fabs(back.ptr<float>()[i] - x.ptr<float>()[i]) <= std::fabs(x.ptr<float>()[i]) / 128.f);
  // parallel_for covers the range exactly once
  std::vector<int> hits(1003, 0);
  parallel_for(0, 1003, 8, [&](int64_t b0, int64_t e0) { for (int64_t i = b0; i < e0; i++) hits[i]++; });
  for (int h : hits) CHECK(h == 1);
  set_nthreads(1);
  CHECK(nthreads() == 1);
  set_nthreads(4);
}

static void test_loader_errors(const std::string& golden) {
  // reference tests/test_sdcpp.cpp:130-143 and tests/test_ovit.cpp:75-85: these must throw
  std::string what;
  CHECK(throws(golden + "/does_not_exist.sdcpp", &what));
  CHECK(what.rfind("sdcpp: cannot open", 0) == 0);
  std::ifstream in(golden + "/tiny_model.sdcpp", std::ios::binary);
  std::string good((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  CHECK(good.size() > 1000);
  auto write = [](const std::string& p, const std::string& d) { std::ofstream o(p, std::ios::binary); o << d; };
  const std::string tmp = "/tmp/sd_b200_dropin_test.sdcpp";
  write(tmp, good.substr(0, good.size() / 2));
  CHECK(throws(tmp, &what) && what == "sdcpp: data out of bounds");
  std::string bad = good; bad[0] = 'X';
  write(tmp, bad);
  CHECK(throws(tmp, &what) && what == "sdcpp: bad magic");
  write(tmp, good.substr(0, 10));
  CHECK(throws(tmp, &what) && what.rfind("sdcpp: truncated file", 0) == 0);
  std::remove(tmp.c_str());
}

static void test_qgemm(int64_t M, int64_t K, int64_t N) {
  // reference tests/test_core.cpp:93-118: qgemm vs fp32 on the dequantized weights, cosine > 0.999
  Tensor A({M, K}, DType::F32), W({N, K}, DType::F32), Wq, sc, out;
  fill_uniform(A, 11);
  fill_uniform(W, 12);
  quantize_rowwise(W, Wq, sc);
  CHECK(Wq.dtype == DType::I8 && Wq.rows() == N && sc.numel() == N);
  qgemm(A, Wq, sc, out);
  CHECK(out.rows() == M && out.cols() == N && out.owning);
  std::vector<float> ref((size_t)M * N);
  for (int64_t i = 0; i < M; i++)
    for (int64_t j = 0; j < N; j++) {
      double s = 0;
      for (int64_t k = 0; k < K; k++)
        s += (double)A.ptr<float>()[i * K + k] * ((float)Wq.ptr<int8_t>()[j * K + k] * sc.ptr<float>()[j]);
      ref[i * N + j] = (float)s;
    }
  const double c = cosine(out.ptr<float>(), ref.data(), M * N);
  std::printf("qgemm %lldx%lldx%lld cosine %.6f\n", (long long)M, (long long)K, (long long)N, c);
  CHECK(c > 0.999);
  for (int64_t i = 0; i < M * N; i++) CHECK(std::isfinite(out.ptr<float>()[i]));
}

static void test_matmul(int64_t M, int64_t K, int64_t N, bool with_bias) {
  // reference tests/test_core.cpp:51-91: matmul vs a naive triple loop, max-abs error / max-abs <= 1e-3
  Tensor A({M, K}, DType::F32), B({K, N}, DType::F32), bias({N}, DType::F32), C;
  fill_uniform(A, 21);
  fill_uniform(B, 22);
  fill_uniform(bias, 23);
  matmul(A, B, C, with_bias ? bias.ptr<float>() : nullptr);
  CHECK(C.rows() == M && C.cols() == N && C.owning);
  double err = 0, mx = 0;
  for (int64_t i = 0; i < M; i++)
    for (int64_t j = 0; j < N; j++) {
      double s = with_bias ? bias.ptr<float>()[j] : 0.0;
      for (int64_t k = 0; k < K; k++) s += (double)A.ptr<float>()[i * K + k] * B.ptr<float>()[k * N + j];
      err = std::max(err, std::fabs(s - C.ptr<float>()[i * N + j]));
      mx = std::max(mx, std::fabs(s));
    }
  std::printf("matmul %lldx%lldx%lld max-abs err / max-abs %.2e\n", (long long)M, (long long)K, (long long)N,
              err / (mx > 0 ? mx : 1));
  CHECK(err <= 1e-3 * (mx > 0 ? mx : 1));
}

static void test_sdpa(int64_t Lq, int64_t Lk, int heads) {
  // reference tests/test_blocks.cpp: attention vs a naive softmax(q k^T / sqrt(hd)) v
  const int64_t hd = 128, C = heads * hd;
  Tensor q({Lq, C}, DType::F32), k({Lk, C}, DType::F32), v({Lk, C}, DType::F32), out;
  fill_uniform(q, 31);
  fill_uniform(k, 32);
  fill_uniform(v, 33);
  blk::sdpa(q, k, v, heads, out);
  CHECK(out.rows() == Lq && out.cols() == C && out.owning);
  double err = 0, mx = 0;
  std::vector<double> s((size_t)Lk);
  for (int h = 0; h < heads; h++)
    for (int64_t i = 0; i < Lq; i++) {
      double m = -1e300, sum = 0;
      for (int64_t j = 0; j < Lk; j++) {
        double d = 0;
        for (int64_t c = 0; c < hd; c++) d += (double)q.ptr<float>()[i * C + h * hd + c] * k.ptr<float>()[j * C + h * hd + c];
        s[j] = d / std::sqrt((double)hd);
        m = std::max(m, s[j]);
      }
      for (int64_t j = 0; j < Lk; j++) { s[j] = std::exp(s[j] - m); sum += s[j]; }
      for (int64_t c = 0; c < hd; c++) {
        double o = 0;
        for (int64_t j = 0; j < Lk; j++) o += s[j] / sum * v.ptr<float>()[j * C + h * hd + c];
        err = std::max(err, std::fabs(o - out.ptr<float>()[i * C + h * hd + c]));
        mx = std::max(mx, std::fabs(o));
      }
    }
  std::printf("sdpa %lldx%lld heads %d max-abs err / max-abs %.2e\n", (long long)Lq, (long long)Lk, heads, err / mx);
  CHECK(err <= 1e-3 * mx);
}

static void test_quantize_rowwise() {
  // reference tests/test_core.cpp:120-132: dequantization error below one scale unit
  Tensor W({37, 513}, DType::F32), Wq, sc;
  fill_uniform(W, 5);
  quantize_rowwise(W, Wq, sc);
  for (int64_t i = 0; i < 37; i++)
    for (int64_t k = 0; k < 513; k++)
      CHECK(std::fabs(Wq.ptr<int8_t>()[i * 513 + k] * sc.ptr<float>()[i] - W.ptr<float>()[i * 513 + k]) < sc.ptr<float>()[i]);
}

static void test_pack(const std::string& golden) {
  // reference tests/test_sdcpp.cpp:56-127 shape of the check: entries, dtypes, scale placement,
  // then the model-side pattern: the scale view sits right after the int8 bytes and qgemm takes
  // the loaded views (src/model/ovi_dit.cpp:30-38,66-70)
  std::shared_ptr<void> owner;
  auto m = load_sdcpp(golden + "/tiny_model.sdcpp", owner);
  CHECK(m.size() == 10);
  const Tensor& w = m.at("blocks.0.ffn.0.weight");
  const Tensor& s = m.at("blocks.0.ffn.0.weight.scale");
  CHECK(w.dtype == DType::I8 && w.rows() == 384 && w.cols() == 256 && !w.owning);
  CHECK(s.dtype == DType::F32 && s.numel() == 384);
  CHECK((const char*)s.data == (const char*)w.data + w.nbytes);
  CHECK(m.at("blocks.0.norm.weight").dtype == DType::F32);
  Tensor A({70, 256}, DType::F32), out;
  fill_uniform(A, 3);
  qgemm(A, w, s, out);                      // served from the device copy made at load
  CHECK(out.rows() == 70 && out.cols() == 384);
  std::vector<float> ref(70 * 384);
  for (int i = 0; i < 70; i++)
    for (int j = 0; j < 384; j++) {
      double acc = 0;
      for (int k = 0; k < 256; k++) acc += (double)A.ptr<float>()[i * 256 + k] * (w.ptr<int8_t>()[j * 256 + k] * s.ptr<float>()[j]);
      ref[i * 384 + j] = (float)acc;
    }
  CHECK(cosine(out.ptr<float>(), ref.data(), 70 * 384) > 0.999);

  // A view of the same bytes with another shape (the caller's i8view2d, src/model/ovi_dit.cpp:42-50,
  // may reshape a pack tensor): [384, 256] seen as [768, 128] with one scale per new row.  The
  // device copy made at load has the pack's own extents; the call must not run with those.
  Tensor v;
  v.shape = {768, 128};
  v.dtype = DType::I8;
  v.data = w.data;
  v.nbytes = w.nbytes;
  v.owning = false;
  Tensor vs({768}, DType::F32), A2({9, 128}, DType::F32), out2;
  for (int j = 0; j < 768; j++) vs.ptr<float>()[j] = 0.01f + 0.001f * (j % 7);
  fill_uniform(A2, 4);
  qgemm(A2, v, vs, out2);
  CHECK(out2.rows() == 9 && out2.cols() == 768);
  std::vector<float> ref2(9 * 768);
  for (int i = 0; i < 9; i++)
    for (int j = 0; j < 768; j++) {
      double acc = 0;
      for (int k = 0; k < 128; k++) acc += (double)A2.ptr<float>()[i * 128 + k] * (v.ptr<int8_t>()[j * 128 + k] * vs.ptr<float>()[j]);
      ref2[i * 768 + j] = (float)acc;
    }
  CHECK(cosine(out2.ptr<float>(), ref2.data(), 9 * 768) > 0.999);
}

static void test_tensor_storage() {
  // Once the device is in use, large owning tensors come from the page-locked pool: still
  // 64-byte aligned, still zero-filled by the public constructor, and a released block that is
  // handed out again is cleared again.
  const int64_t n = 1 << 20;                       // 4 MiB
  void* first = nullptr;
  {
    Tensor t({n}, DType::F32);
    first = t.data;
    CHECK(((uintptr_t)t.data & 63) == 0);
    bool zero = true;
    for (int64_t i = 0; i < n; i += 997) zero = zero && t.ptr<float>()[i] == 0.f;
    CHECK(zero);
    for (int64_t i = 0; i < n; i++) t.ptr<float>()[i] = 1.f;
  }
  Tensor u({n}, DType::F32);
  bool zero = true;
  for (int64_t i = 0; i < n; i += 997) zero = zero && u.ptr<float>()[i] == 0.f;
  CHECK(zero);
  std::printf("tensor storage: block %s\n", u.data == first ? "reused from the pool" : "fresh");
  Tensor small({16}, DType::F32);                  // small tensors stay ordinary allocations
  CHECK(small.owning && ((uintptr_t)small.data & 63) == 0);
}

int main(int argc, char** argv) {
  bool cpu_only = false;
  std::string golden = "tests/golden";
  for (int i = 1; i < argc; i++) {
    if (!std::strcmp(argv[i], "--cpu")) cpu_only = true;
    else golden = argv[i];
  }
  test_containers();
  test_loader_errors(golden);
  if (!cpu_only) {
    test_qgemm(17, 31, 13);
    test_qgemm(64, 1024, 512);
    test_qgemm(300, 3072, 640);
    test_quantize_rowwise();
    test_matmul(17, 31, 13, false);
    test_matmul(64, 1024, 512, true);
    test_matmul(300, 140, 3072, true);
    test_sdpa(70, 130, 2);
    test_sdpa(300, 257, 1);
    test_pack(golden);
    test_tensor_storage();
  }
  if (g_fail) std::printf("test_dropin: %d FAILED\n", g_fail);
  else std::printf("test_dropin: all passed%s\n", cpu_only ? " (cpu part)" : "");
  return g_fail ? 1 : 0;
}
