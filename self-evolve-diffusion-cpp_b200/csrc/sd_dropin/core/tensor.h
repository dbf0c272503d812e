// Declarations of the part of the reference's core API that the B200 drop-in
// library (libsd_b200.so) defines.  The struct layout and the signatures are
// those of the reference's src/core/tensor.h:13-61 -- a program compiled against
// the reference's header links against this library unchanged -- restricted to
// the int8 quantized-linear path: Tensor, the bf16 converters, qgemm,
// quantize_rowwise and the host thread dispatch.  (matmul, silu_inplace, rmsnorm
// and randu of the reference header are not on that path and are not defined here.)
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace sd {

enum class DType : uint8_t { F32 = 0, BF16 = 1, I8 = 2 };

// Row-major host tensor: owning (64-byte aligned, zero-filled) or a view.  Move-only.
struct Tensor {
  std::vector<int64_t> shape;
  DType dtype = DType::F32;
  void* data = nullptr;
  size_t nbytes = 0;
  bool owning = true;

  Tensor() = default;
  Tensor(std::vector<int64_t> s, DType d);
  Tensor(const Tensor&) = delete;
  Tensor& operator=(const Tensor&) = delete;
  Tensor(Tensor&& o) noexcept;
  Tensor& operator=(Tensor&& o) noexcept;
  ~Tensor();

  int64_t numel() const;
  int64_t rows() const { return shape.size() >= 2 ? shape[shape.size() - 2] : 1; }
  int64_t cols() const { return shape.size() >= 1 ? shape[shape.size() - 1] : 1; }
  size_t dim(int i) const { return (size_t)shape[i]; }
  void reshape(std::vector<int64_t> s);  // aborts unless numel is unchanged
  template <typename T> T* ptr() { return reinterpret_cast<T*>(data); }
  template <typename T> const T* ptr() const { return reinterpret_cast<const T*>(data); }
};

void to_f32(const Tensor& bf16, Tensor& out);
void to_bf16(const Tensor& f32, Tensor& out);  // round to nearest even

// out[M,N] = quantized-linear(A[M,K] fp32, Bq[N,K] int8, bs[N] fp32); `out` is replaced by a
// fresh owning tensor.  Runs on the GPU: the device copy of Bq made by load_sdcpp is found by
// Bq.data; a weight that was not loaded from a pack is uploaded for the duration of the call.
void qgemm(const Tensor& A, const Tensor& Bq, const Tensor& bs, Tensor& out);

// W fp32 [N,K] -> Wq int8 [N,K], scale fp32 [N] = absmax/127 (1 for an all-zero row).
void quantize_rowwise(const Tensor& W, Tensor& Wq, Tensor& scale);

// Host-side fork-join over [begin,end) in chunks of `grain`; callers of the path (the bias loop
// of the model code) still use it.
void parallel_for(int64_t begin, int64_t end, int64_t grain,
                  const std::function<void(int64_t, int64_t)>& fn);
int nthreads();
void set_nthreads(int n);

}  // namespace sd
