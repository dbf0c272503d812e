// sdq_qgemm_static_scratch: the quantized linear for callers that must not allocate.
//
// sdq_qgemm keeps the quantized activations (int8 [M,K]) and their row scales in a
// workspace that it grows with cudaMalloc.  Some hosts cannot tolerate that: a
// serving loop that has handed all device memory to its own pool, a plugin running
// inside somebody else's allocator, code between two points where a device-wide
// synchronisation (which cudaMalloc/cudaFree imply) would stall other streams.  For
// them this file holds the same two-kernel sequence with the scratch in a fixed
// array that is part of the library image: it exists on every GPU that loads the
// library, from load until the process exits, whether or not this entry point is
// ever called.
//
// Consequences of the fixed array, all by design:
//   * the problem size is limited (SDQ_STATIC_MAX_ROWS, SDQ_STATIC_MAX_AQ_BYTES);
//     larger calls are rejected with SDQ_ERR_INVALID before anything is launched;
//   * all calls on a device share the one array.  Two calls whose kernels can
//     overlap on the GPU (different streams, no ordering between them) race on
//     it; calls on one stream, or otherwise ordered, are fine;
//   * the array keeps what the last call left.  The activations and scales are
//     overwritten before they are read, so nothing needs clearing between calls.
//     The one word that must be zero for a kernel to record a timed-out wait in it
//     -- the status word -- is zero when the library is loaded and is set back to
//     zero by the host only after a time-out has been reported: a call made
//     with SDQ_SYNC waits for the stream, reads the word and, if a kernel of this or
//     of an earlier call gave up, returns SDQ_ERR_DEVICE_TIMEOUT and clears it.  A
//     caller that never passes SDQ_SYNC never learns of a time-out (the word just
//     stays set); nothing is lost in between, because calls without SDQ_SYNC do not
//     touch it.
//
// The first call on each device performs a one-time set-up on the host (device
// address of the array, kernel attributes, driver entry point).  Make that first
// call outside any stream capture.
#include <cstdio>
#include <mutex>

#include "sdq_internal.h"

namespace {

constexpr size_t kStatusBytes = 256;
constexpr size_t kScaleBytes = (size_t)SDQ_STATIC_MAX_ROWS * sizeof(float);
constexpr size_t kScratchBytes = kStatusBytes + kScaleBytes + (size_t)SDQ_STATIC_MAX_AQ_BYTES;

// [0,256): status word | [256, 256+4*MAX_ROWS): row scales | then the int8 activations.
// In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned char* base = nullptr;  // device address of g_static_scratch on that device
  int sm_count = 0;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_setup_mu;

// One-time, per device, with that device current.
int setup_current_device(int dev, PerDevice** out) {
  std::lock_guard<std::mutex> lk(g_setup_mu);
  PerDevice& d = g_dev[dev];
  if (!d.base) {
    int major = 0, sms = 0;
    SDQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    SDQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10)
      return sdq::fail(SDQ_ERR_CUDA, "sdq_qgemm_static_scratch: this library is built for sm_100a (B200) only");
    std::string why;
    if (int rc = sdq::qgemm_tc_setup(&why)) return sdq::fail(rc, why);
    void* p = nullptr;
    SDQ_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    d.sm_count = sms;
    d.base = static_cast<unsigned char*>(p);
  }
  *out = &d;
  return SDQ_OK;
}

}  // namespace

extern "C" int sdq_qgemm_static_scratch(const int8_t* wq_dev, const float* w_scale_dev, int64_t N,
                                        int64_t K, const float* A_dev, int64_t M, float* out_dev,
                                        const float* bias_dev, uint32_t flags, void* stream) {
  using sdq::fail;
  if (M < 0 || N <= 0 || K <= 0) return fail(SDQ_ERR_INVALID, "sdq_qgemm_static_scratch: bad shape");
  if (flags & (SDQ_A_HOST | SDQ_OUT_HOST))
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_static_scratch: host pointers need staging buffers, which this entry point cannot allocate");
  if (M > SDQ_STATIC_MAX_ROWS || (uint64_t)M * (uint64_t)K > (uint64_t)SDQ_STATIC_MAX_AQ_BYTES)
    return fail(SDQ_ERR_INVALID,
                "sdq_qgemm_static_scratch: M=" + std::to_string(M) + ", K=" + std::to_string(K) +
                    " exceeds the fixed scratch (M <= " + std::to_string(SDQ_STATIC_MAX_ROWS) +
                    ", M*K <= " + std::to_string(SDQ_STATIC_MAX_AQ_BYTES) + "); use sdq_qgemm");
  if (M == 0) return SDQ_OK;
  if (!wq_dev || !w_scale_dev || !A_dev || !out_dev)
    return fail(SDQ_ERR_INVALID, "sdq_qgemm_static_scratch: null pointer");
  int dev = -1;
  SDQ_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(SDQ_ERR_INVALID, "sdq_qgemm_static_scratch: device index out of range");
  PerDevice* d = nullptr;
  if (int rc = setup_current_device(dev, &d)) return rc;

  cudaStream_t s = (cudaStream_t)stream;
  int* status = reinterpret_cast<int*>(d->base);
  float* a_scale = reinterpret_cast<float*>(d->base + kStatusBytes);
  int8_t* aq = reinterpret_cast<int8_t*>(d->base + kStatusBytes + kScaleBytes);

  SDQ_CUDA(sdq::launch_act_quant(A_dev, M, K, aq, a_scale, d->sm_count, s));
  sdq::GemmArgs g;
  g.aq = aq; g.a_scale = a_scale; g.bq = wq_dev; g.b_scale = w_scale_dev; g.bias = bias_dev;
  g.out = out_dev; g.acc_dump = nullptr; g.M = M; g.N = N; g.K = K;
  g.flags = flags & SDQ_GELU_TANH; g.status = status;
  if (!(flags & SDQ_FORCE_SIMT) && sdq::qgemm_tc_supported(g)) {
    std::string why;
    cudaError_t e = sdq::launch_qgemm_tc(g, d->sm_count, s, &why);
    if (e != cudaSuccess)
      return fail(SDQ_ERR_CUDA, why.empty() ? std::string("tcgen05 GEMM launch: ") + cudaGetErrorString(e) : why);
  } else {
    SDQ_CUDA(sdq::launch_qgemm_simt(g, s));
  }
  if (flags & SDQ_SYNC) {
    SDQ_CUDA(cudaStreamSynchronize(s));
    int st = 0;
    SDQ_CUDA(cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
      SDQ_CUDA(cudaMemset(status, 0, sizeof(int)));  // reported: the next time-out can be recorded
      char buf[160];
      snprintf(buf, sizeof buf,
               "sdq_qgemm_static_scratch: a bounded wait inside the GEMM kernel of this or an earlier call gave up (code 0x%x)", st);
      return fail(SDQ_ERR_DEVICE_TIMEOUT, buf);
    }
  }
  return SDQ_OK;
}
