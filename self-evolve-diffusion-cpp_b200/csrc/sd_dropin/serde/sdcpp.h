// .sdcpp v1 loader of the B200 drop-in library; signature of the reference's
// src/serde/sdcpp.h:18-19.
#pragma once
#include <memory>
#include <string>
#include <unordered_map>

#include "core/tensor.h"

namespace sd {

// Maps the file and returns non-owning views: a quantized tensor as `name` (I8, original
// shape) plus `name.scale` (F32 [rows]); a raw tensor as `name` (F32).  Every I8 tensor is
// also uploaded to the GPU once, so that qgemm finds it by the view's data pointer.  `owner`
// keeps the mapping and the device copies alive.  Throws std::runtime_error("sdcpp: ...") on
// a missing, truncated or malformed file.
std::unordered_map<std::string, Tensor> load_sdcpp(const std::string& path,
                                                   std::shared_ptr<void>& owner);

}  // namespace sd
