// B200 drop-in: the .sdcpp v1 pack loader (same signature as the reference project's
// src/serde/sdcpp.h:18-19, so its callers link unchanged).
#pragma once

#include <memory>
#include <string>
#include <unordered_map>

#include "core/tensor.h"

namespace sd {

// Opens and validates `path`, and returns one non-owning Tensor per entry:
//   quantized tensor  ->  "<name>"        I8, the tensor's original shape
//                         "<name>.scale"  F32, one scale per row (row = last dimension)
//   raw tensor        ->  "<name>"        F32
// All views point into a read-only mapping of the file.  In addition every I8 tensor is
// copied to the GPU once, which is how qgemm later finds it from the view's data pointer.
// `owner` holds the mapping and the device copies; keep it alive while the views are in use.
// A missing, truncated or malformed file raises std::runtime_error("sdcpp: ...").
std::unordered_map<std::string, Tensor> load_sdcpp(const std::string& path,
                                                   std::shared_ptr<void>& owner);

}  // namespace sd
