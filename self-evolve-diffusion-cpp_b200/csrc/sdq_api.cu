// C-ABI entry points of libsdq: process/device state, memory helpers, the
// weight registry, and the dispatch of sd::qgemm's two halves onto the kernels.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "sdq_internal.h"

namespace sdq {
namespace {

thread_local std::string t_last_error;
std::atomic<int64_t> g_launches{0};

struct Weight {
  const int8_t* q = nullptr;   // device [N,K]
  const float* scale = nullptr;  // device [N]
  int64_t N = 0, K = 0;
  // an fp32 weight (sdq_fweight_upload): tf32 planes hi / lo, transposed to [N,K]; q is null
  const float* f_hi = nullptr;
  const float* f_lo = nullptr;
  bool owned = false;          // q/scale (or f_hi/f_lo) were allocated by the upload
  const void* host_key = nullptr;
  bool live = false;
};

// Scratch of one stream: quantized activations, their scales, and the staging
// buffers of the host-pointer path.  Grown on demand, never shrunk.
struct Workspace {
  int8_t* aq = nullptr; size_t aq_bytes = 0;
  float* a_scale = nullptr; size_t a_scale_bytes = 0;
  float* a_stage = nullptr; size_t a_stage_bytes = 0;
  float* out_stage = nullptr; size_t out_stage_bytes = 0;
  int32_t* acc = nullptr; size_t acc_bytes = 0;   // split-K partial sums
  float2* ln_stats = nullptr; size_t ln_stats_bytes = 0;  // per-row mean and 1/sqrt(var+eps)
  float* f_split = nullptr; size_t f_split_bytes = 0;     // tf32 planes of the fp32 activations
  float* attn = nullptr; size_t attn_bytes = 0;           // attention: fp16 planes of k, v^T
  // partial int32 sums of the tiles whose K range is shared between CTA pairs (the last, partial
  // wave of the 2-CTA GEMM); all zero between launches: the pass that reads them clears them
  int32_t* tail_acc = nullptr; size_t tail_acc_bytes = 0; uint64_t tail_epoch = 0;
  // the FFN pair's host-pointer pipeline of this stream: two copy streams, events, chunk buffers
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t ev_in[2] = {}, ev_a_free[2] = {}, ev_comp[2] = {}, ev_out_done[2] = {};
  float* pa[2] = {}; size_t pa_bytes[2] = {};
  float* py[2] = {}; size_t py_bytes[2] = {};
  float* ph = nullptr; size_t ph_bytes = 0;
};

// Releases everything a stream's workspace holds (device memory, copy streams, events).
void release_workspace(Workspace& w) {
  cudaFree(w.aq); cudaFree(w.a_scale); cudaFree(w.a_stage); cudaFree(w.out_stage); cudaFree(w.acc);
  cudaFree(w.ln_stats); cudaFree(w.f_split); cudaFree(w.attn); cudaFree(w.tail_acc);
  for (int i = 0; i < 2; i++) {
    cudaFree(w.pa[i]); cudaFree(w.py[i]);
    if (w.ev_in[i]) {
      cudaEventDestroy(w.ev_in[i]); cudaEventDestroy(w.ev_a_free[i]);
      cudaEventDestroy(w.ev_comp[i]); cudaEventDestroy(w.ev_out_done[i]);
    }
  }
  cudaFree(w.ph);
  if (w.copy_in) cudaStreamDestroy(w.copy_in);
  if (w.copy_out) cudaStreamDestroy(w.copy_out);
  w = Workspace();
}

struct Context {
  int device = -1;
  int sm_count = 0;
  int* status = nullptr;  // device word written by a kernel whose bounded wait gave up
  std::mutex mu;
  std::deque<Weight> weights;                        // handle = index + 1 (a deque: no reallocation)
  std::unordered_map<const void*, sdq_weight_t> by_host;
  std::unordered_map<cudaStream_t, Workspace> ws;     // node-based: a Workspace never moves
  std::atomic<uint64_t> tail_epoch{1};                // bumped when a kernel gave up mid-way
  // staged uploads of large weights
  std::mutex upload_mu;
  cudaStream_t up_stream = nullptr;
  void* up_buf[2] = {};
  int up_next = 0;
  cudaEvent_t up_done[2] = {};
};
Context* g_ctx = nullptr;
std::mutex g_init_mu;

template <typename T>
int grow(T** p, size_t* have, size_t need) {
  if (need <= *have) return SDQ_OK;
  if (*p) SDQ_CUDA(cudaFree(*p));
  *p = nullptr; *have = 0;
  // round up so that a slowly growing M does not reallocate every call
  size_t bytes = (need + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(p), bytes);
  if (e != cudaSuccess) return fail(SDQ_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  *have = bytes;
  return SDQ_OK;
}

int need_ctx() {
  if (!g_ctx) return fail(SDQ_ERR_NOT_INIT, "sdq_init has not been called (no CPU fallback exists)");
  return SDQ_OK;
}

// Registry slot of a live handle; the caller holds g_ctx->mu.
Weight* slot_locked(sdq_weight_t h) {
  if (!g_ctx || h == 0 || h > g_ctx->weights.size()) return nullptr;
  Weight* w = &g_ctx->weights[h - 1];
  return w->live ? w : nullptr;
}
// Compute calls work on a copy taken under the lock, so that uploads and releases running
// on other host threads never move or rewrite what a call in progress reads.
struct WeightRef {
  Weight w;
  bool ok = false;
  const Weight* operator->() const { return &w; }
  const Weight& operator*() const { return w; }
  explicit operator bool() const { return ok; }
};
WeightRef get_any_weight(sdq_weight_t h) {
  WeightRef r;
  if (!g_ctx) return r;
  std::lock_guard<std::mutex> lk(g_ctx->mu);
  if (Weight* w = slot_locked(h)) { r.w = *w; r.ok = true; }
  return r;
}
WeightRef get_weight(sdq_weight_t h) {  // an int8 weight
  WeightRef r = get_any_weight(h);
  r.ok = r.ok && r.w.q != nullptr;
  return r;
}
WeightRef get_fweight(sdq_weight_t h) {  // an fp32 weight
  WeightRef r = get_any_weight(h);
  r.ok = r.ok && r.w.f_hi != nullptr;
  return r;
}

int check_status_word() {
  int st = 0;
  SDQ_CUDA(cudaMemcpy(&st, g_ctx->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(g_ctx->status, 0, sizeof(int));
    g_ctx->tail_epoch.fetch_add(1);  // partial sums may be left in the scratch accumulators
    char buf[96];
    snprintf(buf, sizeof buf, "a bounded wait inside the GEMM kernel gave up (code 0x%x)", st);
    return fail(SDQ_ERR_DEVICE_TIMEOUT, buf);
  }
  return SDQ_OK;
}

int run_gemm(const Weight& w, const int8_t* aq, const float* a_scale, int64_t M, float* out,
             const float* bias, int32_t* acc_dump, uint32_t flags, cudaStream_t s,
             const float* residual = nullptr, const float* gate = nullptr) {
  GemmArgs g;
  g.aq = aq; g.a_scale = a_scale; g.bq = w.q; g.b_scale = w.scale; g.bias = bias; g.out = out;
  g.acc_dump = acc_dump; g.M = M; g.N = w.N; g.K = w.K; g.flags = flags & SDQ_GELU_TANH;
  g.status = g_ctx->status;
  g.residual = residual; g.gate = residual ? gate : nullptr;
  if (!(flags & SDQ_FORCE_SIMT) && qgemm_tc_supported(g)) {
    std::string why;
    if (qgemm_tc2_wanted(g, g_ctx->sm_count)) {
      if (qgemm_tc2_tail_tiles(g, g_ctx->sm_count) > 0) {
        // scratch for the partial sums of the shared last wave: zero when first made (and again
        // after a kernel gave up mid-way); every launch that uses it leaves it zero
        Workspace* ws;
        {
          std::lock_guard<std::mutex> lk(g_ctx->mu);
          ws = &g_ctx->ws[s];
        }
        const size_t cap_tiles = (size_t)(g_ctx->sm_count / 2);
        const size_t bytes = cap_tiles * 256 * 256 * sizeof(int32_t);
        const uint64_t epoch = g_ctx->tail_epoch.load();
        if (ws->tail_acc_bytes < bytes || ws->tail_epoch != epoch) {
          if (int rc = grow(&ws->tail_acc, &ws->tail_acc_bytes, bytes)) return rc;
          SDQ_CUDA(cudaMemsetAsync(ws->tail_acc, 0, ws->tail_acc_bytes, s));
          ws->tail_epoch = epoch;
        }
        g.tail_acc = ws->tail_acc;
        g.tail_cap_tiles = (int)cap_tiles;
      }
    }
    const int splits = qgemm_tc_plan_splits(g, g_ctx->sm_count);
    if (splits > 1) {
      Workspace* ws;
      {
        std::lock_guard<std::mutex> lk(g_ctx->mu);
        ws = &g_ctx->ws[s];
      }
      if (int rc = grow(&ws->acc, &ws->acc_bytes, (size_t)M * w.N * 4)) return rc;
      SDQ_CUDA(cudaMemsetAsync(ws->acc, 0, (size_t)M * w.N * 4, s));
      g.splitk_acc = ws->acc;
      g.k_splits = splits;
    }
    cudaError_t e = launch_qgemm_tc(g, g_ctx->sm_count, s, &why);
    if (e != cudaSuccess) return fail(SDQ_ERR_CUDA, why.empty() ? std::string("tcgen05 GEMM launch: ") + cudaGetErrorString(e) : why);
    return SDQ_OK;
  }
  cudaError_t e = launch_qgemm_simt(g, s);
  if (e != cudaSuccess) return fail(SDQ_ERR_CUDA, std::string("SIMT GEMM launch: ") + cudaGetErrorString(e));
  return SDQ_OK;
}

}  // namespace

int fail(int code, const std::string& msg) { t_last_error = msg; return code; }
int cuda_fail(cudaError_t e, const char* what) {
  return fail(SDQ_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// used by the pack loader (sdcpp_file.cpp): page-lock / release a read-only file mapping
bool pin_readonly_mapping(void* base, size_t size) {
  if (!g_ctx || !base || !size) return false;
  cudaError_t e = cudaHostRegister(base, size, cudaHostRegisterReadOnly | cudaHostRegisterPortable);
  if (e != cudaSuccess) {
    cudaGetLastError();  // a refusal is not an error of the load
    return false;
  }
  return true;
}
void unpin_mapping(void* base) {
  if (cudaHostUnregister(base) != cudaSuccess) cudaGetLastError();
}

// used by the pack loader (sdcpp_file.cpp)
int context_sm_count() { return g_ctx ? g_ctx->sm_count : 0; }

}  // namespace sdq

using namespace sdq;

extern "C" {

int sdq_version(void) { return SDQ_VERSION; }
const char* sdq_last_error(void) { return t_last_error.c_str(); }
int sdq_device(void) { return g_ctx ? g_ctx->device : -1; }
int64_t sdq_launch_count(void) { return g_launches.load(); }

int sdq_init(int device) {
  std::lock_guard<std::mutex> lk(g_init_mu);
  if (g_ctx) {
    if (g_ctx->device == device) return SDQ_OK;
    return fail(SDQ_ERR_INVALID, "sdq_init: this process is already bound to another device");
  }
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(SDQ_ERR_CUDA, std::string("no CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "count is 0"));
  if (device < 0 || device >= n) return fail(SDQ_ERR_INVALID, "sdq_init: device index out of range");
  SDQ_CUDA(cudaSetDevice(device));
  cudaDeviceProp p;
  SDQ_CUDA(cudaGetDeviceProperties(&p, device));
  if (p.major != 10)
    return fail(SDQ_ERR_CUDA, "sdq_init: this library is built for sm_100a (B200) only; device is sm_" +
                                  std::to_string(p.major) + std::to_string(p.minor));
  Context* c = new Context;
  c->device = device;
  c->sm_count = p.multiProcessorCount;
  e = cudaMalloc(reinterpret_cast<void**>(&c->status), sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->status, 0, sizeof(int));
  if (e != cudaSuccess) { delete c; return cuda_fail(e, "status word"); }
  std::string why;
  int rc = qgemm_tc_setup(&why);
  if (rc == SDQ_OK) rc = fgemm_setup(&why);
  if (rc == SDQ_OK) rc = sdpa_setup(&why);
  if (rc != SDQ_OK) { cudaFree(c->status); delete c; return fail(rc, why); }
  g_ctx = c;
  return SDQ_OK;
}

int sdq_shutdown(void) {
  std::lock_guard<std::mutex> lk(g_init_mu);
  if (!g_ctx) return SDQ_OK;
  cudaDeviceSynchronize();
  for (auto& w : g_ctx->weights)
    if (w.live && w.owned) {
      cudaFree(const_cast<int8_t*>(w.q)); cudaFree(const_cast<float*>(w.scale));
      cudaFree(const_cast<float*>(w.f_hi)); cudaFree(const_cast<float*>(w.f_lo));
    }
  for (auto& kv : g_ctx->ws) release_workspace(kv.second);
  for (int i = 0; i < 2; i++) {
    if (g_ctx->up_buf[i]) cudaFreeHost(g_ctx->up_buf[i]);
    if (g_ctx->up_done[i]) cudaEventDestroy(g_ctx->up_done[i]);
  }
  if (g_ctx->up_stream) cudaStreamDestroy(g_ctx->up_stream);
  cudaFree(g_ctx->status);
  delete g_ctx;
  g_ctx = nullptr;
  return SDQ_OK;
}

int sdq_int8_mma_probe(int iters, double* seconds, double* tera_ops_per_s) {
  if (int rc = need_ctx()) return rc;
  if (iters < 1 || iters > (1 << 24)) return fail(SDQ_ERR_INVALID, "sdq_int8_mma_probe: iters out of range");
  double sec = 0, ops = 0;
  if (int rc = int8_mma_probe(g_ctx->sm_count, iters, g_ctx->status, &sec, &ops)) return rc;
  if (int rc = check_status_word()) return rc;
  if (seconds) *seconds = sec;
  if (tera_ops_per_s) *tera_ops_per_s = sec > 0 ? ops / sec / 1e12 : 0;
  return SDQ_OK;
}

int sdq_malloc(void** dptr, size_t bytes) {
  if (int rc = need_ctx()) return rc;
  if (!dptr) return fail(SDQ_ERR_INVALID, "sdq_malloc: null out pointer");
  *dptr = nullptr;
  if (bytes == 0) return SDQ_OK;
  cudaError_t e = cudaMalloc(dptr, bytes);
  if (e != cudaSuccess) return fail(SDQ_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  return SDQ_OK;
}
int sdq_free(void* dptr) {
  if (int rc = need_ctx()) return rc;
  if (dptr) SDQ_CUDA(cudaFree(dptr));
  return SDQ_OK;
}
int sdq_malloc_host(void** hptr, size_t bytes) {
  if (int rc = need_ctx()) return rc;
  if (!hptr) return fail(SDQ_ERR_INVALID, "sdq_malloc_host: null out pointer");
  *hptr = nullptr;
  if (bytes == 0) return SDQ_OK;
  cudaError_t e = cudaHostAlloc(hptr, bytes, cudaHostAllocDefault);
  if (e != cudaSuccess) return fail(SDQ_ERR_NOMEM, std::string("cudaHostAlloc: ") + cudaGetErrorString(e));
  return SDQ_OK;
}
int sdq_free_host(void* hptr) {
  if (int rc = need_ctx()) return rc;
  if (hptr) SDQ_CUDA(cudaFreeHost(hptr));
  return SDQ_OK;
}
int sdq_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (bytes) SDQ_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return SDQ_OK;
}
int sdq_selftest_wait_expiry(int limit_ms, int* outcome_dev, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (limit_ms < 1 || limit_ms > 1000)
    return fail(SDQ_ERR_INVALID, "sdq_selftest_wait_expiry: limit_ms must be in 1..1000");
  if (!outcome_dev) return fail(SDQ_ERR_INVALID, "sdq_selftest_wait_expiry: null outcome pointer");
  return wait_expiry_selftest(limit_ms, SDQ_SELFTEST_WAIT_CODE, g_ctx->status, outcome_dev, (cudaStream_t)stream);
}

int sdq_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (bytes) SDQ_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return SDQ_OK;
}
int sdq_memset(void* dst, int value, size_t bytes, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (bytes) SDQ_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
  return SDQ_OK;
}
int sdq_stream_sync(void* stream) {
  if (int rc = need_ctx()) return rc;
  SDQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return check_status_word();
}

int sdq_stream_create(void** stream) {
  if (int rc = need_ctx()) return rc;
  if (!stream) return fail(SDQ_ERR_INVALID, "sdq_stream_create: null out pointer");
  cudaStream_t s = nullptr;
  SDQ_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return SDQ_OK;
}

int sdq_stream_destroy(void* stream) {
  if (int rc = need_ctx()) return rc;
  if (!stream) return SDQ_OK;
  cudaStream_t s = (cudaStream_t)stream;
  SDQ_CUDA(cudaStreamSynchronize(s));
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    auto it = g_ctx->ws.find(s);
    if (it != g_ctx->ws.end()) {
      release_workspace(it->second);
      g_ctx->ws.erase(it);
    }
  }
  SDQ_CUDA(cudaStreamDestroy(s));
  return SDQ_OK;
}

// ---- weights ----
// Host -> device copy of a large pageable (typically file-mapped) range through two pinned
// staging buffers: a few host threads fill one buffer (which is also what pages the file in)
// while the DMA engine drains the other.  Ranges below a threshold take a plain cudaMemcpy.
static int staged_upload(void* dst_dev, const void* src_host, size_t bytes, bool wait_at_end) {
  constexpr size_t kChunk = size_t(32) << 20;
  if (bytes < (size_t(1) << 20)) {
    SDQ_CUDA(cudaMemcpy(dst_dev, src_host, bytes, cudaMemcpyHostToDevice));
    return SDQ_OK;
  }
  Context* c = g_ctx;
  std::lock_guard<std::mutex> lk(c->upload_mu);
  if (!c->up_stream) {
    SDQ_CUDA(cudaStreamCreateWithFlags(&c->up_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; i++) {
      cudaError_t e = cudaHostAlloc(&c->up_buf[i], kChunk, cudaHostAllocDefault);
      if (e != cudaSuccess) return fail(SDQ_ERR_NOMEM, std::string("cudaHostAlloc(staging): ") + cudaGetErrorString(e));
      SDQ_CUDA(cudaEventCreateWithFlags(&c->up_done[i], cudaEventDisableTiming));
    }
  }
  {  // already page-locked (pinned allocation or a registered mapping): direct DMA, no staging
    cudaPointerAttributes pa;
    if (cudaPointerGetAttributes(&pa, src_host) == cudaSuccess && pa.type == cudaMemoryTypeHost) {
      SDQ_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, c->up_stream));
      if (wait_at_end) SDQ_CUDA(cudaStreamSynchronize(c->up_stream));
      return SDQ_OK;
    }
    cudaGetLastError();
  }
  const unsigned hw = std::thread::hardware_concurrency();
  const int nthreads = (int)std::max(1u, std::min(8u, hw ? hw / 2 : 1u));
  size_t off = 0;
  for (; off < bytes; c->up_next ^= 1) {
    const int i = c->up_next;  // buffers alternate across calls too, so uploads of consecutive
                               // tensors of a pack overlap each other's DMA
    const size_t n = std::min(kChunk, bytes - off);
    SDQ_CUDA(cudaEventSynchronize(c->up_done[i]));  // the DMA that last read this buffer is done
    const char* src = static_cast<const char*>(src_host) + off;
    char* dstb = static_cast<char*>(c->up_buf[i]);
    std::vector<std::thread> team;
    const size_t per = (n + nthreads - 1) / nthreads;
    for (int t = 1; t < nthreads; t++) {
      const size_t b = std::min(n, per * t), e = std::min(n, per * (t + 1));
      if (e > b) team.emplace_back([=] { std::memcpy(dstb + b, src + b, e - b); });
    }
    std::memcpy(dstb, src, std::min(n, per));
    for (auto& th : team) th.join();
    SDQ_CUDA(cudaMemcpyAsync(static_cast<char*>(dst_dev) + off, dstb, n, cudaMemcpyHostToDevice, c->up_stream));
    SDQ_CUDA(cudaEventRecord(c->up_done[i], c->up_stream));
    off += n;
  }
  if (wait_at_end) SDQ_CUDA(cudaStreamSynchronize(c->up_stream));
  return SDQ_OK;
}

static int register_weight(const Weight& w, sdq_weight_t* out) {
  std::lock_guard<std::mutex> lk(g_ctx->mu);
  g_ctx->weights.push_back(w);
  *out = (sdq_weight_t)g_ctx->weights.size();
  if (w.host_key) g_ctx->by_host[w.host_key] = *out;
  return SDQ_OK;
}

static int weight_upload_impl(const int8_t* q_host, const float* scale_host, int64_t N, int64_t K,
                              sdq_weight_t* out, bool wait_at_end) {
  if (int rc = need_ctx()) return rc;
  if (!q_host || !scale_host || !out || N <= 0 || K <= 0)
    return fail(SDQ_ERR_INVALID, "sdq_weight_upload: null pointer or non-positive shape");
  int8_t* dq = nullptr; float* ds = nullptr;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&dq), (size_t)N * K);  // cudaMalloc is >= 256-B aligned
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ds), (size_t)N * 4);
  if (e == cudaSuccess) e = cudaMemcpy(ds, scale_host, (size_t)N * 4, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) { cudaFree(dq); cudaFree(ds); return cuda_fail(e, "sdq_weight_upload"); }
  if (int rc = staged_upload(dq, q_host, (size_t)N * K, wait_at_end)) { cudaFree(dq); cudaFree(ds); return rc; }
  Weight w; w.q = dq; w.scale = ds; w.N = N; w.K = K; w.owned = true; w.host_key = q_host; w.live = true;
  return register_weight(w, out);
}

int sdq_weight_upload(const int8_t* q_host, const float* scale_host, int64_t N, int64_t K,
                      sdq_weight_t* out) {
  return weight_upload_impl(q_host, scale_host, N, K, out, true);
}

int sdq_weight_wrap_device(const int8_t* q_dev, const float* scale_dev, int64_t N, int64_t K,
                           sdq_weight_t* out) {
  if (int rc = need_ctx()) return rc;
  if (!q_dev || !scale_dev || !out || N <= 0 || K <= 0)
    return fail(SDQ_ERR_INVALID, "sdq_weight_wrap_device: null pointer or non-positive shape");
  Weight w; w.q = q_dev; w.scale = scale_dev; w.N = N; w.K = K; w.owned = false; w.live = true;
  return register_weight(w, out);
}

int sdq_weight_lookup(const void* q_host, sdq_weight_t* out) {
  if (int rc = need_ctx()) return rc;
  if (!out) return fail(SDQ_ERR_INVALID, "sdq_weight_lookup: null out pointer");
  std::lock_guard<std::mutex> lk(g_ctx->mu);
  auto it = g_ctx->by_host.find(q_host);
  if (it == g_ctx->by_host.end()) { *out = 0; return fail(SDQ_ERR_NOT_FOUND, "sdq_weight_lookup: no weight was uploaded from this host address"); }
  *out = it->second;
  return SDQ_OK;
}

int sdq_weight_info(sdq_weight_t h, int64_t* N, int64_t* K, const int8_t** q_dev,
                    const float** scale_dev) {
  if (int rc = need_ctx()) return rc;
  WeightRef w = get_any_weight(h);  // an fp32 weight reports q_dev = scale_dev = NULL
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_weight_info: bad weight handle");
  if (N) *N = w->N;
  if (K) *K = w->K;
  if (q_dev) *q_dev = w->q;
  if (scale_dev) *scale_dev = w->scale;
  return SDQ_OK;
}

int sdq_weight_release(sdq_weight_t h) {
  if (int rc = need_ctx()) return rc;
  std::lock_guard<std::mutex> lk(g_ctx->mu);
  Weight* w = slot_locked(h);
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_weight_release: bad weight handle");
  if (w->owned) {
    cudaFree(const_cast<int8_t*>(w->q)); cudaFree(const_cast<float*>(w->scale));
    cudaFree(const_cast<float*>(w->f_hi)); cudaFree(const_cast<float*>(w->f_lo));
  }
  if (w->host_key) {
    auto it = g_ctx->by_host.find(w->host_key);
    if (it != g_ctx->by_host.end() && it->second == h) g_ctx->by_host.erase(it);
  }
  *w = Weight();
  return SDQ_OK;
}

// ---- hot path ----
int sdq_quantize_activations(const float* A_dev, int64_t M, int64_t K, int8_t* aq_dev,
                             float* a_scale_dev, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (M < 0 || K < 0) return fail(SDQ_ERR_INVALID, "sdq_quantize_activations: negative shape");
  if (M == 0 || K == 0) return SDQ_OK;
  if (!A_dev || !aq_dev || !a_scale_dev) return fail(SDQ_ERR_INVALID, "sdq_quantize_activations: null pointer");
  SDQ_CUDA(launch_act_quant(A_dev, M, K, aq_dev, a_scale_dev, g_ctx->sm_count, (cudaStream_t)stream));
  return SDQ_OK;
}

// Scratch for the exact row statistics of stream s, or null when tree sums were asked for.
static int ln_stats_for(cudaStream_t s, int64_t M, uint32_t flags, float2** out) {
  *out = nullptr;
  if (flags & SDQ_LN_TREE_SUMS) return SDQ_OK;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  if (int rc = grow(&ws->ln_stats, &ws->ln_stats_bytes, (size_t)M * sizeof(float2))) return rc;
  *out = ws->ln_stats;
  return SDQ_OK;
}

int sdq_layernorm_mod_quantize(const float* X_dev, int64_t M, int64_t K, const float* shift_dev,
                               const float* scale_dev, float eps, int8_t* aq_dev,
                               float* a_scale_dev, float* h_out_dev, uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (M < 0 || K < 0) return fail(SDQ_ERR_INVALID, "sdq_layernorm_mod_quantize: negative shape");
  if (M == 0 || K == 0) return SDQ_OK;
  if (!X_dev || !shift_dev || !scale_dev || !aq_dev || !a_scale_dev)
    return fail(SDQ_ERR_INVALID, "sdq_layernorm_mod_quantize: null pointer");
  float2* stats;
  if (int rc = ln_stats_for((cudaStream_t)stream, M, flags, &stats)) return rc;
  cudaError_t e = launch_ln_mod_quant(X_dev, M, K, shift_dev, scale_dev, eps, aq_dev, a_scale_dev,
                                      h_out_dev, stats, (flags & SDQ_LN_AFFINE) ? 1 : 0,
                                      g_ctx->sm_count, (cudaStream_t)stream);
  if (e == cudaErrorInvalidValue)
    return fail(SDQ_ERR_INVALID, "sdq_layernorm_mod_quantize: needs K % 4 == 0, K <= 16384 and 16-byte aligned pointers");
  SDQ_CUDA(e);
  return SDQ_OK;
}

int sdq_qgemm_prequantized(sdq_weight_t h, const int8_t* aq_dev, const float* a_scale_dev,
                           int64_t M, float* out_dev, const float* bias_dev,
                           int32_t* acc_dump_dev, uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w = get_weight(h);
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_qgemm_prequantized: bad weight handle");
  if (M < 0) return fail(SDQ_ERR_INVALID, "sdq_qgemm_prequantized: negative M");
  if (M == 0) return SDQ_OK;
  if (!aq_dev || !a_scale_dev || !out_dev) return fail(SDQ_ERR_INVALID, "sdq_qgemm_prequantized: null pointer");
  int rc = run_gemm(*w, aq_dev, a_scale_dev, M, out_dev, bias_dev, acc_dump_dev, flags, (cudaStream_t)stream);
  if (rc == SDQ_OK && (flags & SDQ_SYNC)) rc = sdq_stream_sync(stream);
  return rc;
}

int sdq_qgemm(sdq_weight_t h, const float* A, int64_t M, float* out, const float* bias,
              uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w = get_weight(h);
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_qgemm: bad weight handle");
  if (M < 0) return fail(SDQ_ERR_INVALID, "sdq_qgemm: negative M");
  if (M == 0) return SDQ_OK;
  if (!A || !out) return fail(SDQ_ERR_INVALID, "sdq_qgemm: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t N = w->N, K = w->K;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  if (int rc = grow(&ws->aq, &ws->aq_bytes, (size_t)M * K)) return rc;
  if (int rc = grow(&ws->a_scale, &ws->a_scale_bytes, (size_t)M * 4)) return rc;
  const float* A_dev = A;
  float* out_dev = out;
  if (flags & SDQ_A_HOST) {
    if (int rc = grow(&ws->a_stage, &ws->a_stage_bytes, (size_t)M * K * 4)) return rc;
    SDQ_CUDA(cudaMemcpyAsync(ws->a_stage, A, (size_t)M * K * 4, cudaMemcpyHostToDevice, s));
    A_dev = ws->a_stage;
  }
  if (flags & SDQ_OUT_HOST) {
    if (int rc = grow(&ws->out_stage, &ws->out_stage_bytes, (size_t)M * N * 4)) return rc;
    out_dev = ws->out_stage;
  }
  SDQ_CUDA(launch_act_quant(A_dev, M, K, ws->aq, ws->a_scale, g_ctx->sm_count, s));
  if (int rc = run_gemm(*w, ws->aq, ws->a_scale, M, out_dev, bias, nullptr, flags, s)) return rc;
  if (flags & SDQ_OUT_HOST) {
    SDQ_CUDA(cudaMemcpyAsync(out, out_dev, (size_t)M * N * 4, cudaMemcpyDeviceToHost, s));
    // the caller owns `out` when this returns: a host result must be complete
    return sdq_stream_sync(stream);
  }
  if (flags & SDQ_SYNC) return sdq_stream_sync(stream);
  return SDQ_OK;
}

// ---- fp32 linears ----
int sdq_fweight_upload(const float* w, int64_t K, int64_t N, uint32_t flags, sdq_weight_t* out) {
  if (int rc = need_ctx()) return rc;
  if (!w || !out || K <= 0 || N <= 0)
    return fail(SDQ_ERR_INVALID, "sdq_fweight_upload: null pointer or non-positive shape");
  const size_t bytes = (size_t)K * N * 4;
  float* src = nullptr;
  float *hi = nullptr, *lo = nullptr;
  cudaError_t e = cudaSuccess;
  if (flags & SDQ_A_HOST) {
    e = cudaMalloc(reinterpret_cast<void**>(&src), bytes);
    if (e == cudaSuccess) e = cudaMemcpy(src, w, bytes, cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&hi), bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&lo), bytes);
  if (e == cudaSuccess) e = launch_transpose_split(src ? src : w, K, N, hi, lo, nullptr);
  if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
  cudaFree(src);
  if (e != cudaSuccess) {
    cudaFree(hi); cudaFree(lo);
    return fail(e == cudaErrorMemoryAllocation ? SDQ_ERR_NOMEM : SDQ_ERR_CUDA,
                std::string("sdq_fweight_upload: ") + cudaGetErrorString(e));
  }
  Weight wt; wt.f_hi = hi; wt.f_lo = lo; wt.N = N; wt.K = K; wt.owned = true; wt.live = true;
  if (flags & SDQ_A_HOST) wt.host_key = w;
  return register_weight(wt, out);
}

int sdq_fmatmul(sdq_weight_t h, const float* A, int64_t M, float* out, const float* bias_dev,
                uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w = get_fweight(h);
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_fmatmul: bad weight handle (not an fp32 weight)");
  if (M < 0) return fail(SDQ_ERR_INVALID, "sdq_fmatmul: negative M");
  if (M == 0) return SDQ_OK;
  if (!A || !out) return fail(SDQ_ERR_INVALID, "sdq_fmatmul: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t N = w->N, K = w->K;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  if (int rc = grow(&ws->f_split, &ws->f_split_bytes, (size_t)M * K * 8)) return rc;
  const float* A_dev = A;
  float* out_dev = out;
  if (flags & SDQ_A_HOST) {
    if (int rc = grow(&ws->a_stage, &ws->a_stage_bytes, (size_t)M * K * 4)) return rc;
    SDQ_CUDA(cudaMemcpyAsync(ws->a_stage, A, (size_t)M * K * 4, cudaMemcpyHostToDevice, s));
    A_dev = ws->a_stage;
  }
  if (flags & SDQ_OUT_HOST) {
    if (int rc = grow(&ws->out_stage, &ws->out_stage_bytes, (size_t)M * N * 4)) return rc;
    out_dev = ws->out_stage;
  }
  std::string why;
  cudaError_t e = launch_fmatmul(A_dev, M, K, w->f_hi, w->f_lo, N, bias_dev, out_dev, ws->f_split,
                                 ws->f_split + (size_t)M * K, g_ctx->status, flags, g_ctx->sm_count, s, &why);
  if (e != cudaSuccess)
    return fail(SDQ_ERR_CUDA, why.empty() ? std::string("fp32 GEMM launch: ") + cudaGetErrorString(e) : why);
  if (flags & SDQ_OUT_HOST) {
    SDQ_CUDA(cudaMemcpyAsync(out, out_dev, (size_t)M * N * 4, cudaMemcpyDeviceToHost, s));
    return sdq_stream_sync(stream);
  }
  return (flags & SDQ_SYNC) ? sdq_stream_sync(stream) : SDQ_OK;
}

// ---- attention ----
int sdq_sdpa(const float* q_dev, const float* k_dev, const float* v_dev, int64_t Lq, int64_t Lk,
             int64_t C, int heads, float* out_dev, uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (Lq < 0 || Lk < 0 || C <= 0 || heads <= 0 || C % heads != 0)
    return fail(SDQ_ERR_INVALID, "sdq_sdpa: bad shape (C must be a positive multiple of heads)");
  if (flags & (SDQ_A_HOST | SDQ_OUT_HOST)) return fail(SDQ_ERR_INVALID, "sdq_sdpa: device pointers only");
  if (Lq == 0) return SDQ_OK;
  if (!q_dev || !out_dev || (Lk > 0 && (!k_dev || !v_dev))) return fail(SDQ_ERR_INVALID, "sdq_sdpa: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  if (int rc = grow(&ws->attn, &ws->attn_bytes, sdpa_scratch_bytes(Lq, Lk, C, heads) + 16)) return rc;
  std::string why;
  cudaError_t e = launch_sdpa(q_dev, k_dev, v_dev, Lq, Lk, C, heads, out_dev, ws->attn, g_ctx->status, flags,
                              g_ctx->sm_count, s, &why);
  if (e != cudaSuccess)
    return fail(SDQ_ERR_CUDA, why.empty() ? std::string("attention launch: ") + cudaGetErrorString(e) : why);
  return (flags & SDQ_SYNC) ? sdq_stream_sync(stream) : SDQ_OK;
}

int sdq_qgemm_residual(sdq_weight_t h, const float* A_dev, int64_t M, const float* residual_dev,
                       const float* gate_dev, float* out_dev, const float* bias_dev,
                       uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w = get_weight(h);
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_qgemm_residual: bad weight handle");
  if (M < 0) return fail(SDQ_ERR_INVALID, "sdq_qgemm_residual: negative M");
  if (flags & (SDQ_A_HOST | SDQ_OUT_HOST))
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_residual: device pointers only");
  if (M == 0) return SDQ_OK;
  if (!A_dev || !residual_dev || !out_dev) return fail(SDQ_ERR_INVALID, "sdq_qgemm_residual: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  if (int rc = grow(&ws->aq, &ws->aq_bytes, (size_t)M * w->K)) return rc;
  if (int rc = grow(&ws->a_scale, &ws->a_scale_bytes, (size_t)M * 4)) return rc;
  SDQ_CUDA(launch_act_quant(A_dev, M, w->K, ws->aq, ws->a_scale, g_ctx->sm_count, s));
  if (int rc = run_gemm(*w, ws->aq, ws->a_scale, M, out_dev, bias_dev, nullptr, flags, s, residual_dev, gate_dev))
    return rc;
  return (flags & SDQ_SYNC) ? sdq_stream_sync(stream) : SDQ_OK;
}

// ---- column split across GPUs ----
int sdq_ipc_export(const void* dptr, unsigned char handle[64]) {
  if (int rc = need_ctx()) return rc;
  if (!dptr || !handle) return fail(SDQ_ERR_INVALID, "sdq_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  SDQ_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(dptr)));
  std::memcpy(handle, &h, 64);
  return SDQ_OK;
}

int sdq_ipc_open(const unsigned char handle[64], void** dptr) {
  if (int rc = need_ctx()) return rc;
  if (!dptr || !handle) return fail(SDQ_ERR_INVALID, "sdq_ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  SDQ_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SDQ_OK;
}

int sdq_ipc_close(void* dptr) {
  if (int rc = need_ctx()) return rc;
  if (dptr) SDQ_CUDA(cudaIpcCloseMemHandle(dptr));
  return SDQ_OK;
}

int sdq_qgemm_colsplit(sdq_weight_t h, const float* A_dev, int64_t M, int64_t col0, int64_t N_total,
                       float* const* outs_dev, int n_outs, const float* bias_dev, uint32_t flags,
                       void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w = get_weight(h);
  if (!w) return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: bad weight handle");
  if (M < 0 || col0 < 0 || N_total < col0 + w->N || n_outs < 1 || n_outs > 8 || !outs_dev)
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: bad shape or destination count (1..8)");
  if (col0 % 32 != 0 || (w->N % 32 != 0 && col0 + w->N != N_total))
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: a column block must start on a multiple of 32 and, unless it is the last one, be a multiple of 32 wide");
  if (N_total % 4 != 0 || w->K % 16 != 0)
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: needs N_total % 4 == 0 and K % 16 == 0");
  if (M == 0) return SDQ_OK;
  if (!A_dev) return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  if (int rc = grow(&ws->aq, &ws->aq_bytes, (size_t)M * w->K)) return rc;
  if (int rc = grow(&ws->a_scale, &ws->a_scale_bytes, (size_t)M * 4)) return rc;
  SDQ_CUDA(launch_act_quant(A_dev, M, w->K, ws->aq, ws->a_scale, g_ctx->sm_count, s));
  GemmArgs g;
  g.aq = ws->aq; g.a_scale = ws->a_scale; g.bq = w->q; g.b_scale = w->scale; g.bias = bias_dev;
  g.out = outs_dev[0]; g.acc_dump = nullptr; g.M = M; g.N = w->N; g.K = w->K;
  g.flags = flags & SDQ_GELU_TANH; g.status = g_ctx->status;
  g.out_col0 = col0; g.out_ld = N_total; g.out_copies = n_outs;
  for (int i = 0; i < n_outs; i++) {
    if (!outs_dev[i]) return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: null destination");
    g.out_all[i] = outs_dev[i];
  }
  if (!qgemm_tc_supported(g))
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_colsplit: the tensor-core kernel cannot take this problem (K % 16 != 0, "
                                 "an operand that is not 16-byte aligned, or a dimension of 2^31 or more)");
  if (const char* unfit = qgemm_tc2_unfit(g))
    return fail(SDQ_ERR_INVALID, std::string("sdq_qgemm_colsplit: ") + unfit);
  std::string why;
  cudaError_t e = launch_qgemm_tc2(g, g_ctx->sm_count, s, &why);
  if (e != cudaSuccess) return fail(SDQ_ERR_CUDA, why.empty() ? std::string("column-split GEMM launch: ") + cudaGetErrorString(e) : why);
  return (flags & SDQ_SYNC) ? sdq_stream_sync(stream) : SDQ_OK;
}

// ---- FFN pair ----
// fc1 -> GELU(tanh) -> fc2 on [r0, r1) rows that are already on the device.
static int ffn_rows_device(const Weight& w1, const float* b1, const Weight& w2, const float* b2,
                           const float* x, int64_t rows, float* h, float* y, Workspace* ws,
                           cudaStream_t s) {
  if (int rc = grow(&ws->aq, &ws->aq_bytes, (size_t)rows * std::max(w1.K, w2.K))) return rc;
  if (int rc = grow(&ws->a_scale, &ws->a_scale_bytes, (size_t)rows * 4)) return rc;
  SDQ_CUDA(launch_act_quant(x, rows, w1.K, ws->aq, ws->a_scale, g_ctx->sm_count, s));
  if (int rc = run_gemm(w1, ws->aq, ws->a_scale, rows, h, b1, nullptr, SDQ_GELU_TANH, s)) return rc;
  SDQ_CUDA(launch_act_quant(h, rows, w2.K, ws->aq, ws->a_scale, g_ctx->sm_count, s));
  return run_gemm(w2, ws->aq, ws->a_scale, rows, y, b2, nullptr, 0, s);
}

int sdq_ffn_pair(sdq_weight_t h1, const float* bias1_dev, sdq_weight_t h2, const float* bias2_dev,
                 const float* x, int64_t M, float* hidden_dev, float* y, uint32_t flags,
                 void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w1 = get_weight(h1);
  WeightRef w2 = get_weight(h2);
  if (!w1 || !w2) return fail(SDQ_ERR_INVALID, "sdq_ffn_pair: bad weight handle");
  if (w2->K != w1->N) return fail(SDQ_ERR_INVALID, "sdq_ffn_pair: fc2 input width differs from fc1 output width");
  if (M < 0) return fail(SDQ_ERR_INVALID, "sdq_ffn_pair: negative M");
  if (M == 0) return SDQ_OK;
  if (!x || !y) return fail(SDQ_ERR_INVALID, "sdq_ffn_pair: null pointer");
  const bool x_host = flags & SDQ_A_HOST, y_host = flags & SDQ_OUT_HOST;
  if (x_host != y_host) return fail(SDQ_ERR_INVALID, "sdq_ffn_pair: x and y must both be host or both be device memory");
  cudaStream_t s = (cudaStream_t)stream;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  const int64_t D = w1->K, F = w1->N, Dout = w2->N;
  if (!x_host) {
    float* h = hidden_dev;
    if (!h) {  // caller does not want the hidden activations: keep them in the staging buffer
      if (int rc = grow(&ws->out_stage, &ws->out_stage_bytes, (size_t)M * F * 4)) return rc;
      h = ws->out_stage;
    }
    if (int rc = ffn_rows_device(*w1, bias1_dev, *w2, bias2_dev, x, M, h, y, ws, s)) return rc;
    return (flags & SDQ_SYNC) ? sdq_stream_sync(stream) : SDQ_OK;
  }

  // Host x and y: rows are independent, so the pair is run chunk by chunk with the
  // copies of neighbouring chunks overlapping the arithmetic:
  //   copy_in : H2D x[i+1]   |  stream : quant, fc1, quant, fc2 on chunk i  |  copy_out : D2H y[i-1]
  // The pipeline's streams, events and chunk buffers belong to the caller's stream, like the
  // rest of its scratch: calls on different streams share nothing.
  Workspace* c = ws;
  if (!c->copy_in) {
    SDQ_CUDA(cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking));
    SDQ_CUDA(cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; i++) {
      SDQ_CUDA(cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming));
      SDQ_CUDA(cudaEventCreateWithFlags(&c->ev_a_free[i], cudaEventDisableTiming));
      SDQ_CUDA(cudaEventCreateWithFlags(&c->ev_comp[i], cudaEventDisableTiming));
      SDQ_CUDA(cudaEventCreateWithFlags(&c->ev_out_done[i], cudaEventDisableTiming));
    }
  }
  // rows per chunk: small enough that the first upload and the last download (which nothing
  // overlaps) are short, large enough that each chunk's GEMMs still fill the GPU
  static const int64_t chunk_rows = [] {
    const char* v = std::getenv("SDQ_FFN_CHUNK_ROWS");
    const int64_t n = v ? std::atoll(v) : 0;
    return n >= 128 ? n : 2048;
  }();
  const int64_t chunk = std::min<int64_t>(M, chunk_rows);
  for (int i = 0; i < 2; i++) {
    if (int rc = grow(&c->pa[i], &c->pa_bytes[i], (size_t)chunk * D * 4)) return rc;
    if (int rc = grow(&c->py[i], &c->py_bytes[i], (size_t)chunk * Dout * 4)) return rc;
  }
  if (int rc = grow(&c->ph, &c->ph_bytes, (size_t)chunk * F * 4)) return rc;
  // the copy streams start after whatever the caller already queued on `stream`
  SDQ_CUDA(cudaEventRecord(c->ev_comp[0], s));
  SDQ_CUDA(cudaStreamWaitEvent(c->copy_in, c->ev_comp[0], 0));
  SDQ_CUDA(cudaStreamWaitEvent(c->copy_out, c->ev_comp[0], 0));
  int64_t n = 0;
  for (int64_t r0 = 0; r0 < M; r0 += chunk, n++) {
    const int64_t rows = std::min(chunk, M - r0);
    const int b = (int)(n & 1);
    if (n >= 2) SDQ_CUDA(cudaStreamWaitEvent(c->copy_in, c->ev_a_free[b], 0));  // x buffer consumed
    SDQ_CUDA(cudaMemcpyAsync(c->pa[b], x + r0 * D, (size_t)rows * D * 4, cudaMemcpyHostToDevice, c->copy_in));
    SDQ_CUDA(cudaEventRecord(c->ev_in[b], c->copy_in));
    SDQ_CUDA(cudaStreamWaitEvent(s, c->ev_in[b], 0));
    if (n >= 2) SDQ_CUDA(cudaStreamWaitEvent(s, c->ev_out_done[b], 0));         // y buffer copied out
    if (int rc = ffn_rows_device(*w1, bias1_dev, *w2, bias2_dev, c->pa[b], rows, c->ph, c->py[b], ws, s)) return rc;
    SDQ_CUDA(cudaEventRecord(c->ev_a_free[b], s));
    SDQ_CUDA(cudaEventRecord(c->ev_comp[b], s));
    SDQ_CUDA(cudaStreamWaitEvent(c->copy_out, c->ev_comp[b], 0));
    SDQ_CUDA(cudaMemcpyAsync(y + r0 * Dout, c->py[b], (size_t)rows * Dout * 4, cudaMemcpyDeviceToHost, c->copy_out));
    SDQ_CUDA(cudaEventRecord(c->ev_out_done[b], c->copy_out));
  }
  // the caller's stream (and the host) see the call as complete when the last copy-out is
  SDQ_CUDA(cudaStreamWaitEvent(s, c->ev_out_done[0], 0));
  SDQ_CUDA(cudaStreamWaitEvent(s, c->ev_out_done[1], 0));
  SDQ_CUDA(cudaStreamSynchronize(c->copy_out));
  return sdq_stream_sync(stream);
}

int sdq_ffn_block(sdq_weight_t h1, const float* bias1_dev, sdq_weight_t h2, const float* bias2_dev,
                  float* x_dev, int64_t M, const float* shift_dev, const float* scale_dev,
                  const float* gate_dev, float eps, uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  WeightRef w1 = get_weight(h1);
  WeightRef w2 = get_weight(h2);
  if (!w1 || !w2) return fail(SDQ_ERR_INVALID, "sdq_ffn_block: bad weight handle");
  if (w2->K != w1->N) return fail(SDQ_ERR_INVALID, "sdq_ffn_block: fc2 input width differs from fc1 output width");
  if (w2->N != w1->K) return fail(SDQ_ERR_INVALID, "sdq_ffn_block: fc2 output width differs from the width of x");
  if (M < 0) return fail(SDQ_ERR_INVALID, "sdq_ffn_block: negative M");
  if (flags & (SDQ_A_HOST | SDQ_OUT_HOST)) return fail(SDQ_ERR_INVALID, "sdq_ffn_block: device pointers only");
  if (M == 0) return SDQ_OK;
  if (!x_dev || !shift_dev || !scale_dev || !gate_dev) return fail(SDQ_ERR_INVALID, "sdq_ffn_block: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  Workspace* ws;
  {
    std::lock_guard<std::mutex> lk(g_ctx->mu);
    ws = &g_ctx->ws[s];
  }
  const int64_t D = w1->K, F = w1->N;
  if (int rc = grow(&ws->aq, &ws->aq_bytes, (size_t)M * std::max(D, F))) return rc;
  if (int rc = grow(&ws->a_scale, &ws->a_scale_bytes, (size_t)M * 4)) return rc;
  if (int rc = grow(&ws->out_stage, &ws->out_stage_bytes, (size_t)M * F * 4)) return rc;
  float* hbuf = ws->out_stage;
  // layernorm + modulation + quantization of x in one pass: fp32 h is never written
  float2* stats;
  if (int rc = ln_stats_for(s, M, flags, &stats)) return rc;
  cudaError_t e = launch_ln_mod_quant(x_dev, M, D, shift_dev, scale_dev, eps, ws->aq, ws->a_scale,
                                      nullptr, stats, 0, g_ctx->sm_count, s);
  if (e == cudaErrorInvalidValue)
    return fail(SDQ_ERR_INVALID, "sdq_ffn_block: needs a width with K % 4 == 0, K <= 16384 and 16-byte aligned pointers");
  SDQ_CUDA(e);
  if (int rc = run_gemm(*w1, ws->aq, ws->a_scale, M, hbuf, bias1_dev, nullptr, SDQ_GELU_TANH, s)) return rc;
  SDQ_CUDA(launch_act_quant(hbuf, M, F, ws->aq, ws->a_scale, g_ctx->sm_count, s));
  // fc2 + bias, then x += y * gate in the same epilogue (x is read and written in place)
  if (int rc = run_gemm(*w2, ws->aq, ws->a_scale, M, x_dev, bias2_dev, nullptr, 0, s, x_dev, gate_dev)) return rc;
  return (flags & SDQ_SYNC) ? sdq_stream_sync(stream) : SDQ_OK;
}

// ---- weight quantizers ----
static size_t src_elem_size(int dt) { return dt == SDQ_F32 ? 4 : 2; }

int sdq_quantize_rows(const void* src, int src_dtype, int64_t rows, int64_t last, int mode,
                      int8_t* q, float* scale, uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (rows < 0 || last < 0) return fail(SDQ_ERR_INVALID, "sdq_quantize_rows: negative shape");
  if (src_dtype != SDQ_F32 && src_dtype != SDQ_BF16 && src_dtype != SDQ_F16)
    return fail(SDQ_ERR_INVALID, "sdq_quantize_rows: unknown source dtype");
  if (mode != SDQ_MODE_PACKER && mode != SDQ_MODE_ROWWISE)
    return fail(SDQ_ERR_INVALID, "sdq_quantize_rows: unknown mode");
  if (mode == SDQ_MODE_ROWWISE && src_dtype != SDQ_F32)
    return fail(SDQ_ERR_INVALID, "sdq_quantize_rows: the rowwise recipe takes fp32 input only");
  if (rows == 0 || last == 0) return SDQ_OK;
  if (!src || !q || !scale) return fail(SDQ_ERR_INVALID, "sdq_quantize_rows: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t numel = (size_t)rows * last, in_bytes = numel * src_elem_size(src_dtype);
  void* d_src = nullptr; int8_t* d_q = nullptr; float* d_scale = nullptr;
  const void* k_src = src; int8_t* k_q = q; float* k_scale = scale;
  int rc = SDQ_OK;
  cudaError_t e = cudaSuccess;
  if (flags & SDQ_SRC_HOST) {
    e = cudaMalloc(&d_src, in_bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_src, src, in_bytes, cudaMemcpyHostToDevice, s);
    k_src = d_src;
  }
  if (e == cudaSuccess && (flags & SDQ_DST_HOST)) {
    e = cudaMalloc(reinterpret_cast<void**>(&d_q), numel);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d_scale), (size_t)rows * 4);
    k_q = d_q; k_scale = d_scale;
  }
  if (e == cudaSuccess)
    e = launch_quantize_rows(k_src, src_dtype, rows, last, mode, k_q, k_scale, g_ctx->sm_count, s);
  if (e == cudaSuccess && (flags & SDQ_DST_HOST)) {
    e = cudaMemcpyAsync(q, d_q, numel, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(scale, d_scale, (size_t)rows * 4, cudaMemcpyDeviceToHost, s);
  }
  if (e == cudaSuccess && (flags & (SDQ_SRC_HOST | SDQ_DST_HOST))) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) rc = cuda_fail(e, "sdq_quantize_rows");
  cudaFree(d_src); cudaFree(d_q); cudaFree(d_scale);
  return rc;
}

int sdq_dequant_rows(const int8_t* q, const float* scale, int64_t rows, int64_t last, float* w,
                     uint32_t flags, void* stream) {
  if (int rc = need_ctx()) return rc;
  if (rows < 0 || last < 0) return fail(SDQ_ERR_INVALID, "sdq_dequant_rows: negative shape");
  if (rows == 0 || last == 0) return SDQ_OK;
  if (!q || !scale || !w) return fail(SDQ_ERR_INVALID, "sdq_dequant_rows: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t numel = (size_t)rows * last;
  int8_t* d_q = nullptr; float* d_scale = nullptr; float* d_w = nullptr;
  const int8_t* k_q = q; const float* k_scale = scale; float* k_w = w;
  cudaError_t e = cudaSuccess;
  if (flags & SDQ_SRC_HOST) {
    e = cudaMalloc(reinterpret_cast<void**>(&d_q), numel);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d_scale), (size_t)rows * 4);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_q, q, numel, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_scale, scale, (size_t)rows * 4, cudaMemcpyHostToDevice, s);
    k_q = d_q; k_scale = d_scale;
  }
  if (e == cudaSuccess && (flags & SDQ_DST_HOST)) {
    e = cudaMalloc(reinterpret_cast<void**>(&d_w), numel * 4);
    k_w = d_w;
  }
  if (e == cudaSuccess) e = launch_dequant_rows(k_q, k_scale, rows, last, k_w, g_ctx->sm_count, s);
  if (e == cudaSuccess && (flags & SDQ_DST_HOST)) e = cudaMemcpyAsync(w, d_w, numel * 4, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess && (flags & (SDQ_SRC_HOST | SDQ_DST_HOST))) e = cudaStreamSynchronize(s);
  int rc = e == cudaSuccess ? SDQ_OK : cuda_fail(e, "sdq_dequant_rows");
  cudaFree(d_q); cudaFree(d_scale); cudaFree(d_w);
  return rc;
}

}  // extern "C"

namespace sdq {
// Pack loader: upload without waiting for the DMA of each tensor; pack_upload_finish() waits once.
int pack_upload_weight(const int8_t* q_host, const float* scale_host, int64_t N, int64_t K,
                       sdq_weight_t* out) {
  return weight_upload_impl(q_host, scale_host, N, K, out, false);
}
int pack_upload_finish() {
  if (g_ctx && g_ctx->up_stream) SDQ_CUDA(cudaStreamSynchronize(g_ctx->up_stream));
  return SDQ_OK;
}
}  // namespace sdq
