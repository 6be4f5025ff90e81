// TEST INFRASTRUCTURE: see ../framework/op_kernel.h.  Declarations of the tensor-format helpers the shim calls.
#pragma once
#include <string>
#include <vector>

#include "tensorflow/core/framework/op_kernel.h"

namespace tensorflow {
enum TensorFormat { FORMAT_NHWC = 0, FORMAT_NCHW = 1 };
bool FormatFromString(const std::string &format_str, TensorFormat *format);
template <typename T> T GetTensorDim(const std::vector<T> &attributes, TensorFormat format, char dimension);
int64 GetTensorDim(const Tensor &tensor, TensorFormat format, char dimension);
TensorShape ShapeFromFormat(TensorFormat format, int64 N, int64 H, int64 W, int64 C);
}  // namespace tensorflow
