// B200 drop-in: declarations for the int8 quantized-linear path.
//
// libsd_b200.so defines these symbols.  Object code built against the reference project's
// own core header (src/core/tensor.h:13-61) links against it unchanged: the Tensor object has
// the same members in the same order and every function has the same mangled name.  Only the
// part of that header which lies on the linear path is provided -- the tensor container, bf16
// conversion, qgemm, quantize_rowwise, the fp32 matmul and the host thread dispatch; silu,
// rmsnorm and the test RNG are not on the path and are not defined here.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace sd {

// Element types; the numeric values are part of the binary interface (F32 0, BF16 1, I8 2).
enum class DType : uint8_t { F32 = 0, BF16 = 1, I8 = 2 };

// Host tensor, row-major.  Either owns its storage (64-byte aligned, zero-filled on
// construction, released on destruction) or is a view of memory owned elsewhere
// (`owning == false`).  Movable, not copyable.
struct Tensor {
  // --- data members: order and types fixed by the binary interface ---
  std::vector<int64_t> shape;
  DType dtype = DType::F32;
  void* data = nullptr;
  size_t nbytes = 0;
  bool owning = true;

  // --- construction / lifetime ---
  Tensor() = default;
  Tensor(std::vector<int64_t> dims, DType type);  // owning, zero-filled
  ~Tensor();
  Tensor(Tensor&& other) noexcept;
  Tensor& operator=(Tensor&& other) noexcept;
  Tensor(const Tensor&) = delete;
  Tensor& operator=(const Tensor&) = delete;

  // --- shape queries ---
  int64_t numel() const;
  // second-to-last extent (1 for rank < 2) and last extent (1 for rank 0)
  int64_t rows() const {
    const size_t r = shape.size();
    return r < 2 ? 1 : shape[r - 2];
  }
  int64_t cols() const { return shape.empty() ? 1 : shape.back(); }
  size_t dim(int axis) const { return static_cast<size_t>(shape[axis]); }
  void reshape(std::vector<int64_t> dims);  // element count must not change (aborts otherwise)

  // --- typed access ---
  template <typename T>
  T* ptr() {
    return static_cast<T*>(data);
  }
  template <typename T>
  const T* ptr() const {
    return static_cast<const T*>(data);
  }
};

// bf16 <-> fp32; the narrowing rounds to nearest even.
void to_bf16(const Tensor& f32, Tensor& out);
void to_f32(const Tensor& bf16, Tensor& out);

// Quantized linear on the GPU.
//   A  fp32 [M,K] activations      Bq int8 [N,K] weights, one row per output channel
//   bs fp32 [N] weight scales      out fp32 [M,N], replaced by a freshly allocated tensor
// Each row of A is quantized to int8 by its own absmax, the products are accumulated in int32
// and rescaled by a_scale[i] * bs[j].  The device copy of Bq that load_sdcpp made is found by
// Bq.data; a weight that did not come from a pack is uploaded for the duration of the call.
void qgemm(const Tensor& A, const Tensor& Bq, const Tensor& bs, Tensor& out);

// The fp32 linear on the GPU: C[M,N] = A[M,K] * B[K,N] (+ bias[N]); C is replaced by a freshly
// allocated tensor.  A and B are fp32 or bf16 (widened first).  B is looked up by B.data among
// the weights already on the device and otherwise uploaded for the duration of the call.
// Three tf32 tensor-core products per fp32 product: within the reference's matmul tolerance,
// not bit-identical to any particular CPU summation order.
void matmul(const Tensor& A, const Tensor& B, Tensor& C, const float* bias = nullptr);

// fp32 [N,K] weights -> int8 [N,K] and one scale per row (absmax / 127; 1 for an all-zero row).
void quantize_rowwise(const Tensor& W, Tensor& Wq, Tensor& scale);

// Host-side fork-join used by callers around the path (e.g. the model's bias loop):
// fn(b, e) over [begin, end) in pieces of `grain`.
int nthreads();
void set_nthreads(int n);
void parallel_for(int64_t begin, int64_t end, int64_t grain,
                  const std::function<void(int64_t, int64_t)>& fn);

}  // namespace sd
