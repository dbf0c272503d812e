// B200 drop-in: the attention entry of the reference's block library.
//
// Only the function that sits between the quantized projections of a DiT block is provided:
// scaled-dot-product attention (the reference declares it in src/model/blocks.h:60-66 with the
// same name, namespace and argument order, so object code built against that header links
// against libsd_b200.so unchanged).  Layer norms, RoPE and the Linear container of that header
// are host-side code of the caller and are not defined here.
#pragma once

#include "core/tensor.h"

namespace sd {
namespace blk {

// out[Lq,C] = softmax(q k^T / sqrt(C / num_heads)) v for every head; q fp32 [Lq,C], k and v fp32
// [Lk,C]; out is replaced by a freshly allocated tensor.  `causal` is accepted for signature
// compatibility and must be false (the reference never sets it).  Runs on the GPU through
// sdq_sdpa: inside the reference's 1e-3 tolerance, not bit-identical to a CPU summation order.
void sdpa(const Tensor& q, const Tensor& k, const Tensor& v, int num_heads, Tensor& out,
          bool causal = false);

}  // namespace blk
}  // namespace sd
