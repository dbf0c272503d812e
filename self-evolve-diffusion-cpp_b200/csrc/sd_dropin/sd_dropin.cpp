// libsd_b200.so: the reference's sd:: functions of the int8 quantized-linear path,
// defined on top of the sdq C ABI (include/sdq.h).  Host-side container code
// (Tensor, bf16 conversion, parallel_for) is plain C++; everything that computes
// goes to the GPU through libsdq.so and throws when that fails -- there is no CPU
// implementation of qgemm or quantize_rowwise in this library.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <thread>
#include <unordered_map>

#include "core/tensor.h"
#include "model/blocks.h"
#include "sdq.h"
#include "serde/sdcpp.h"

namespace sd {
namespace {

size_t elem_size(DType d) { return d == DType::F32 ? 4 : d == DType::BF16 ? 2 : 1; }

std::atomic<bool> g_device_ready{false};

void ensure_device() {
  static std::once_flag once;
  static int rc = SDQ_OK;
  static std::string msg;
  std::call_once(once, [] {
    const char* dev = std::getenv("SD_DEVICE");
    rc = sdq_init(dev ? std::atoi(dev) : 0);
    if (rc != SDQ_OK) msg = sdq_last_error();
    else g_device_ready.store(true);
  });
  if (rc != SDQ_OK) throw std::runtime_error("sd (B200): " + msg);
}

[[noreturn]] void raise_last() { throw std::runtime_error(sdq_last_error()); }

// Storage of owning tensors.  The caller of the reference's interface allocates a fresh
// output for every linear (src/core/qgemm.cpp:75) and hands activations over as plain host
// tensors; copies between pageable memory and the GPU run at a fraction of the PCIe rate and
// block the host.  Once the device is in use, blocks of 256 KiB and more therefore come from
// page-locked memory, and because page-locking costs far more than a copy, released blocks
// are kept and handed out again (the forward pass asks for the same few sizes over and over).
// SD_PINNED_POOL_MB bounds the idle blocks kept (default 8192; 0 switches the pool off).
class PinnedPool {
 public:
  void* get(size_t bytes) {
    if (!g_device_ready.load() || bytes < kMinBytes || cap() == 0) return nullptr;
    const size_t want = (bytes + kGrain - 1) / kGrain * kGrain;
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = idle_.lower_bound(want);
      if (it != idle_.end() && it->first <= want + want / 8) {
        void* p = it->second;
        live_[p] = it->first;
        idle_bytes_ -= it->first;
        idle_.erase(it);
        return p;
      }
    }
    void* p = nullptr;
    if (sdq_malloc_host(&p, want) != SDQ_OK || !p) return nullptr;  // the caller falls back to malloc
    std::lock_guard<std::mutex> lk(mu_);
    live_[p] = want;
    return p;
  }
  // true when p was a block of this pool (and has been taken back)
  bool put(void* p) {
    size_t size = 0;
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = live_.find(p);
      if (it == live_.end()) return false;
      size = it->second;
      live_.erase(it);
      if (idle_bytes_ + size <= cap()) {
        idle_.emplace(size, p);
        idle_bytes_ += size;
        return true;
      }
    }
    sdq_free_host(p);
    return true;
  }

 private:
  static constexpr size_t kMinBytes = size_t(256) << 10, kGrain = size_t(1) << 20;
  static size_t cap() {
    static const size_t c = [] {
      const char* v = std::getenv("SD_PINNED_POOL_MB");
      return (size_t)(v ? std::atoll(v) : 8192) << 20;
    }();
    return c;
  }
  std::mutex mu_;
  std::unordered_map<void*, size_t> live_;
  std::multimap<size_t, void*> idle_;
  size_t idle_bytes_ = 0;
};
PinnedPool& pool() {
  static PinnedPool* p = new PinnedPool;  // never destroyed: tensors may outlive static teardown
  return *p;
}

void* tensor_alloc(size_t nbytes) {
  if (void* p = pool().get(nbytes)) return p;
  void* p = aligned_alloc(64, (nbytes + 63) / 64 * 64 + 64);
  if (!p) throw std::bad_alloc();
  return p;
}
void tensor_free(void* p) {
  if (p && !pool().put(p)) std::free(p);
}

// An owning tensor whose bytes are NOT cleared: for results that are overwritten in full.
Tensor uninitialized(std::vector<int64_t> shape, DType d) {
  Tensor t;
  int64_t n = 1;
  for (int64_t x : shape) n *= x;
  t.shape = std::move(shape);
  t.dtype = d;
  t.nbytes = (size_t)n * elem_size(d);
  t.data = tensor_alloc(t.nbytes);
  t.owning = true;
  return t;
}

}  // namespace

// ---- Tensor (reference src/core/tensor.cpp:19-37) ----
Tensor::Tensor(std::vector<int64_t> s, DType d) : shape(std::move(s)), dtype(d) {
  int64_t n = 1;
  for (int64_t x : shape) n *= x;
  nbytes = (size_t)n * elem_size(dtype);
  data = tensor_alloc(nbytes);
  std::memset(data, 0, nbytes);
}
Tensor::~Tensor() {
  if (owning && data) tensor_free(data);
}
Tensor::Tensor(Tensor&& o) noexcept { *this = std::move(o); }
Tensor& Tensor::operator=(Tensor&& o) noexcept {
  if (this == &o) return *this;
  if (owning && data) tensor_free(data);
  shape = std::move(o.shape);
  dtype = o.dtype;
  data = o.data;
  nbytes = o.nbytes;
  owning = o.owning;
  o.data = nullptr;
  o.nbytes = 0;
  return *this;
}
int64_t Tensor::numel() const {
  int64_t n = 1;
  for (int64_t x : shape) n *= x;
  return n;
}
void Tensor::reshape(std::vector<int64_t> s) {
  int64_t n = 1;
  for (int64_t x : s) n *= x;
  if (n != numel()) std::abort();
  shape = std::move(s);
}

// ---- bf16 (reference src/core/tensor.cpp:39-60) ----
void to_f32(const Tensor& bf16, Tensor& out) {
  out = Tensor(bf16.shape, DType::F32);
  const uint16_t* s = bf16.ptr<uint16_t>();
  uint32_t* d = out.ptr<uint32_t>();
  for (int64_t i = 0, n = bf16.numel(); i < n; i++) d[i] = (uint32_t)s[i] << 16;
}
void to_bf16(const Tensor& f32, Tensor& out) {
  out = Tensor(f32.shape, DType::BF16);
  const uint32_t* s = f32.ptr<uint32_t>();
  uint16_t* d = out.ptr<uint16_t>();
  for (int64_t i = 0, n = f32.numel(); i < n; i++) {
    uint32_t u = s[i];
    u += 0x7fffu + ((u >> 16) & 1u);
    d[i] = (uint16_t)(u >> 16);
  }
}

// ---- the hot path (reference src/core/qgemm.cpp:73-142) ----
void qgemm(const Tensor& A, const Tensor& Bq, const Tensor& bs, Tensor& out) {
  const int64_t M = A.rows(), K = A.cols(), N = Bq.rows();
  if (M == 0 || N == 0 || K == 0) {  // an empty problem gives a zero tensor (src/core/qgemm.cpp:75-76)
    out = Tensor({M, N}, DType::F32);
    return;
  }
  ensure_device();
  out = uninitialized({M, N}, DType::F32);  // every element is written by the copy back
  sdq_weight_t w = 0;
  bool temporary = false;
  // The device copy made at load time is the pack tensor viewed as [numel / last, last]; a
  // caller's view of the same bytes with another shape (i8view2d, src/model/ovi_dit.cpp:42-50)
  // must not run with the cached extents.
  int64_t wn = 0, wk = 0;
  if (sdq_weight_lookup(Bq.data, &w) != SDQ_OK || sdq_weight_info(w, &wn, &wk, nullptr, nullptr) != SDQ_OK ||
      wn != N || wk != K) {
    if (sdq_weight_upload(Bq.ptr<int8_t>(), bs.ptr<float>(), N, K, &w) != SDQ_OK) raise_last();
    temporary = true;
  }
  const int rc = sdq_qgemm(w, A.ptr<float>(), M, out.ptr<float>(), nullptr,
                           SDQ_A_HOST | SDQ_OUT_HOST, nullptr);
  const std::string msg = rc != SDQ_OK ? sdq_last_error() : "";
  if (temporary) sdq_weight_release(w);
  if (rc != SDQ_OK) throw std::runtime_error(msg);
}

// ---- the fp32 linear (reference src/core/gemm.cpp:115-160) ----
void matmul(const Tensor& A, const Tensor& B, Tensor& C, const float* bias) {
  Tensor Af, Bf;
  const Tensor* a = &A;
  const Tensor* b = &B;
  if (A.dtype == DType::BF16) { to_f32(A, Af); a = &Af; }
  if (B.dtype == DType::BF16) { to_f32(B, Bf); b = &Bf; }
  const int64_t M = a->rows(), K = a->cols(), N = b->cols();
  C = (M == 0 || N == 0 || K == 0) ? Tensor({M, N}, DType::F32) : uninitialized({M, N}, DType::F32);
  if (M == 0 || N == 0) return;
  if (K == 0) {  // an empty sum: only the bias is left, as in the reference
    if (bias)
      for (int64_t i = 0; i < M; i++) std::memcpy(C.ptr<float>() + i * N, bias, (size_t)N * 4);
    return;
  }
  ensure_device();
  sdq_weight_t w = 0;
  bool temporary = false;
  int64_t wn = 0, wk = 0;
  const int8_t* wq = nullptr;
  // a resident copy only counts when it is an fp32 weight of exactly this shape
  if (b != &B || sdq_weight_lookup(B.data, &w) != SDQ_OK ||
      sdq_weight_info(w, &wn, &wk, &wq, nullptr) != SDQ_OK || wq != nullptr || wn != N || wk != K) {
    if (sdq_fweight_upload(b->ptr<float>(), K, N, SDQ_A_HOST, &w) != SDQ_OK) raise_last();
    temporary = true;
  }
  float* bias_dev = nullptr;
  int rc = SDQ_OK;
  if (bias) {
    rc = sdq_malloc(reinterpret_cast<void**>(&bias_dev), (size_t)N * 4);
    if (rc == SDQ_OK) rc = sdq_memcpy_h2d(bias_dev, bias, (size_t)N * 4, nullptr);
  }
  if (rc == SDQ_OK)
    rc = sdq_fmatmul(w, a->ptr<float>(), M, C.ptr<float>(), bias_dev, SDQ_A_HOST | SDQ_OUT_HOST, nullptr);
  const std::string msg = rc != SDQ_OK ? sdq_last_error() : "";
  if (bias_dev) sdq_free(bias_dev);
  if (temporary) sdq_weight_release(w);
  if (rc != SDQ_OK) throw std::runtime_error(msg);
}

// ---- attention (reference src/model/blocks.cpp:113-199) ----
namespace blk {
void sdpa(const Tensor& q, const Tensor& k, const Tensor& v, int num_heads, Tensor& out, bool causal) {
  if (causal) throw std::runtime_error("sd (B200): causal attention is not provided (the reference never uses it)");
  const int64_t Lq = q.rows(), Lk = k.rows(), C = q.cols();
  out = Tensor({Lq, C}, DType::F32);
  if (Lq == 0 || C == 0) return;
  ensure_device();
  const size_t qb = (size_t)Lq * C * 4, kb = (size_t)Lk * C * 4;
  float *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
  int rc = sdq_malloc(reinterpret_cast<void**>(&dq), qb);
  if (rc == SDQ_OK) rc = sdq_malloc(reinterpret_cast<void**>(&dout), qb);
  if (rc == SDQ_OK && kb) rc = sdq_malloc(reinterpret_cast<void**>(&dk), kb);
  if (rc == SDQ_OK && kb) rc = sdq_malloc(reinterpret_cast<void**>(&dv), kb);
  if (rc == SDQ_OK) rc = sdq_memcpy_h2d(dq, q.data, qb, nullptr);
  if (rc == SDQ_OK && kb) rc = sdq_memcpy_h2d(dk, k.data, kb, nullptr);
  if (rc == SDQ_OK && kb) rc = sdq_memcpy_h2d(dv, v.data, kb, nullptr);
  if (rc == SDQ_OK) rc = sdq_sdpa(dq, dk, dv, Lq, Lk, C, num_heads, dout, 0, nullptr);
  if (rc == SDQ_OK) rc = sdq_memcpy_d2h(out.data, dout, qb, nullptr);
  if (rc == SDQ_OK) rc = sdq_stream_sync(nullptr);
  const std::string msg = rc != SDQ_OK ? sdq_last_error() : "";
  sdq_free(dq); sdq_free(dk); sdq_free(dv); sdq_free(dout);
  if (rc != SDQ_OK) throw std::runtime_error(msg);
}
}  // namespace blk

// reference src/core/tensor.cpp:63-78
void quantize_rowwise(const Tensor& W, Tensor& Wq, Tensor& scale) {
  const int64_t N = W.rows(), K = W.cols();
  Wq = Tensor({N, K}, DType::I8);
  scale = Tensor({N}, DType::F32);
  if (N == 0 || K == 0) return;
  ensure_device();
  if (sdq_quantize_rows(W.data, SDQ_F32, N, K, SDQ_MODE_ROWWISE, Wq.ptr<int8_t>(),
                        scale.ptr<float>(), SDQ_SRC_HOST | SDQ_DST_HOST, nullptr) != SDQ_OK)
    raise_last();
}

// reference src/serde/sdcpp.cpp:47-133
std::unordered_map<std::string, Tensor> load_sdcpp(const std::string& path,
                                                   std::shared_ptr<void>& owner) {
  // Format errors are reported before a device is required, as the reference would.
  sdq_pack* probe = nullptr;
  if (sdq_pack_open(path.c_str(), 0, &probe) != SDQ_OK) raise_last();
  sdq_pack_close(probe);
  ensure_device();
  sdq_pack* p = nullptr;
  if (sdq_pack_open(path.c_str(), SDQ_PACK_UPLOAD, &p) != SDQ_OK) raise_last();
  owner = std::shared_ptr<void>(p, [](void* q) { sdq_pack_close(static_cast<sdq_pack*>(q)); });
  std::unordered_map<std::string, Tensor> out;
  for (int64_t i = 0, n = sdq_pack_count(p); i < n; i++) {
    sdq_entry e;
    if (sdq_pack_entry(p, i, &e) != SDQ_OK) raise_last();
    Tensor t;
    t.shape.assign(e.dims, e.dims + e.ndim);
    t.dtype = e.dtype == SDQ_DT_I8 ? DType::I8 : DType::F32;
    t.data = const_cast<void*>(e.data);
    t.nbytes = (size_t)e.nbytes;
    t.owning = false;
    out.emplace(e.name, std::move(t));
  }
  return out;
}

// ---- host thread dispatch (reference src/core/tensor.cpp:81-103) ----
namespace {
std::atomic<int> g_threads{(int)std::thread::hardware_concurrency()};
}
int nthreads() { return g_threads.load(); }
void set_nthreads(int n) { g_threads.store(n > 0 ? n : 1); }

void parallel_for(int64_t begin, int64_t end, int64_t grain,
                  const std::function<void(int64_t, int64_t)>& fn) {
  if (end <= begin) return;
  if (grain < 1) grain = 1;
  const int64_t chunks = (end - begin + grain - 1) / grain;
  int nt = nthreads();
  if (chunks < nt) nt = (int)chunks;
  if (nt <= 1) {
    fn(begin, end);
    return;
  }
  std::atomic<int64_t> next{0};
  auto work = [&] {
    for (int64_t c = next.fetch_add(1); c < chunks; c = next.fetch_add(1)) {
      const int64_t b = begin + c * grain;
      fn(b, b + grain < end ? b + grain : end);
    }
  };
  std::vector<std::thread> team;
  team.reserve(nt - 1);
  for (int t = 1; t < nt; t++) team.emplace_back(work);
  work();
  for (auto& th : team) th.join();
}

}  // namespace sd
