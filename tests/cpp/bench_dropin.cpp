// Wall-clock cost of one DiT FFN through the drop-in library exactly as the reference's
// caller runs it (src/model/ovi_dit.cpp:214-222 with mlin of :66-84): weights come from a
// .sdcpp pack opened with sd::load_sdcpp, activations are host sd::Tensor objects, and a step is
//     sd::qgemm(x, fc1) -> bias pass on the host -> GELU on the host -> sd::qgemm(h, fc2) -> bias pass
// with a freshly allocated output tensor per linear.  Prints one JSON object on stdout.
//
//   bench_dropin <rows> <steps> [<scratch directory>]
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "core/tensor.h"
#include "serde/sdcpp.h"

using namespace sd;
using Clock = std::chrono::steady_clock;

static double ms_since(Clock::time_point t0) {
  return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

static uint64_t g_rng = 0x243f6a8885a308d3ull;
static inline uint64_t next_u64() {
  g_rng ^= g_rng << 13; g_rng ^= g_rng >> 7; g_rng ^= g_rng << 17;
  return g_rng;
}

// One quantized entry of a .sdcpp v1 file: int8 [n,k] bytes followed by n fp32 scales.
static void append_weight(std::vector<char>& blob, int64_t n, int64_t k) {
  const size_t at = blob.size();
  blob.resize(at + (size_t)n * k + (size_t)n * 4);
  int8_t* q = reinterpret_cast<int8_t*>(blob.data() + at);
  for (int64_t i = 0; i < n * k; i += 8) {
    uint64_t r = next_u64();
    for (int j = 0; j < 8 && i + j < n * k; j++, r >>= 8) q[i + j] = (int8_t)((int)(r & 0xff) % 255 - 127);
  }
  std::vector<float> sc((size_t)n);
  for (auto& s : sc) s = 1e-4f + 1e-4f * (float)(next_u64() & 1023) / 1024.f;
  std::memcpy(blob.data() + at + (size_t)n * k, sc.data(), (size_t)n * 4);
}

static void put_entry(std::ofstream& f, const std::string& name, int64_t n, int64_t k, uint64_t off) {
  const uint32_t nl = (uint32_t)name.size(), nd = 2;
  const uint8_t dt = 0;
  f.write((const char*)&nl, 4); f.write(name.data(), nl); f.write((const char*)&dt, 1);
  f.write((const char*)&nd, 4); f.write((const char*)&n, 8); f.write((const char*)&k, 8);
  f.write((const char*)&off, 8);
}

// y[i,j] += b[j]: the separate pass mlin runs after qgemm (src/model/ovi_dit.cpp:71-79)
static void bias_pass(Tensor& y, const std::vector<float>& b) {
  const int64_t M = y.rows(), N = y.cols();
  float* yp = y.ptr<float>();
  parallel_for(0, M, 32, [&](int64_t s, int64_t e) {
    for (int64_t i = s; i < e; i++)
      for (int64_t j = 0; j < N; j++) yp[i * N + j] += b[j];
  });
}
// gelu_tanh_inplace (src/model/ovi_dit.cpp:132-142)
static void gelu_pass(Tensor& x) {
  const int64_t n = x.numel();
  float* p = x.ptr<float>();
  parallel_for(0, n, 4096, [&](int64_t b, int64_t e) {
    for (int64_t i = b; i < e; i++) {
      const float v = p[i], u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      p[i] = 0.5f * v * (1.f + std::tanh(u));
    }
  });
}

int main(int argc, char** argv) {
  const int64_t M = argc > 1 ? std::atoll(argv[1]) : 27280;
  const int steps = argc > 2 ? std::atoi(argv[2]) : 2;
  const std::string dir = argc > 3 ? argv[3] : "/tmp";
  const int64_t D = 3072, F = 14336;
  const std::string path = dir + "/sdq_bench_dropin.sdcpp";
  {
    std::vector<char> blob;
    blob.reserve((size_t)2 * D * F + (size_t)(D + F) * 4);
    append_weight(blob, F, D);
    const uint64_t off2 = blob.size();
    append_weight(blob, D, F);
    std::ofstream f(path, std::ios::binary);
    const uint32_t ver = 1, cnt = 2;
    f.write("SDCP", 4); f.write((const char*)&ver, 4); f.write((const char*)&cnt, 4);
    put_entry(f, "ffn.0.weight", F, D, 0);
    put_entry(f, "ffn.2.weight", D, F, off2);
    f.write(blob.data(), (std::streamsize)blob.size());
    if (!f) { std::fprintf(stderr, "cannot write %s\n", path.c_str()); return 2; }
  }
  try {
    std::shared_ptr<void> owner;
    auto t_load = Clock::now();
    auto pack = load_sdcpp(path, owner);
    const double load_ms = ms_since(t_load);
    const Tensor& w1 = pack.at("ffn.0.weight");
    const Tensor& s1 = pack.at("ffn.0.weight.scale");
    const Tensor& w2 = pack.at("ffn.2.weight");
    const Tensor& s2 = pack.at("ffn.2.weight.scale");
    std::vector<float> b1((size_t)F), b2((size_t)D);
    for (auto& v : b1) v = 0.02f * ((float)(next_u64() & 2047) / 1024.f - 1.f);
    for (auto& v : b2) v = 0.02f * ((float)(next_u64() & 2047) / 1024.f - 1.f);

    auto make_x = [&] {
      Tensor x({M, D}, DType::F32);
      float* p = x.ptr<float>();
      parallel_for(0, M * D, 1 << 16, [&](int64_t b, int64_t e) {
        uint64_t s = 0x9e3779b97f4a7c15ull ^ (uint64_t)b * 0xd1342543de82ef95ull;
        for (int64_t i = b; i < e; i++) {
          s ^= s << 13; s ^= s >> 7; s ^= s << 17;
          p[i] = 0.5f * ((float)(int32_t)(s >> 40) / 8388608.f - 1.f);
        }
      });
      return x;
    };
    double t_q1 = 0, t_host = 0, t_q2 = 0, t_total = 0;
    double checksum = 0;
    for (int it = 0; it < steps + 1; it++) {  // step 0 is the warm-up (first touch of every buffer size)
      Tensor x = make_x();                    // like the caller's activations: a fresh host tensor
      Tensor h, y;
      auto t0 = Clock::now();
      qgemm(x, w1, s1, h);
      auto t1 = Clock::now();
      bias_pass(h, b1);
      gelu_pass(h);
      auto t2 = Clock::now();
      qgemm(h, w2, s2, y);
      bias_pass(y, b2);
      auto t3 = Clock::now();
      if (it > 0) {
        t_q1 += std::chrono::duration<double, std::milli>(t1 - t0).count();
        t_host += std::chrono::duration<double, std::milli>(t2 - t1).count();
        t_q2 += std::chrono::duration<double, std::milli>(t3 - t2).count();
        t_total += std::chrono::duration<double, std::milli>(t3 - t0).count();
      }
      checksum += (double)y.ptr<float>()[0] + (double)y.ptr<float>()[y.numel() - 1];
    }
    const double ms = t_total / steps;
    const double ops = 2.0 * 2.0 * (double)M * D * F;
    const char* pool = std::getenv("SD_PINNED_POOL_MB");
    std::printf(
        "{\"rows\": %lld, \"steps\": %d, \"ms_per_step\": %.3f, \"tops\": %.3f, \"qgemm_fc1_ms\": %.3f, "
        "\"host_bias_gelu_ms\": %.3f, \"qgemm_fc2_plus_bias_ms\": %.3f, \"pack_load_ms\": %.1f, "
        "\"host_threads\": %d, \"pinned_pool_mb\": \"%s\", \"h2d_bytes_per_step\": %lld, "
        "\"d2h_bytes_per_step\": %lld, \"checksum\": %.6g}\n",
        (long long)M, steps, ms, ops / (ms * 1e-3) / 1e12, t_q1 / steps, t_host / steps, t_q2 / steps, load_ms,
        nthreads(), pool ? pool : "default", (long long)(4 * M * (D + F)), (long long)(4 * M * (D + F)), checksum);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "bench_dropin: %s\n", e.what());
    std::remove(path.c_str());
    return 1;
  }
  std::remove(path.c_str());
  return 0;
}
