// TEST INFRASTRUCTURE: see ../framework/op_kernel.h.  The tensor-format helpers the shim calls, with the meaning
// TensorFlow gives them for 4-D tensors.
#pragma once
#include <string>
#include <vector>

#include "tensorflow/core/framework/op_kernel.h"

namespace tensorflow {
enum TensorFormat { FORMAT_NHWC = 0, FORMAT_NCHW = 1 };
inline bool FormatFromString(const std::string &format_str, TensorFormat *format)
{
    if (format_str == "NHWC") { *format = FORMAT_NHWC; return true; }
    if (format_str == "NCHW") { *format = FORMAT_NCHW; return true; }
    return false;
}
inline int DimIndex(TensorFormat format, char dimension)
{
    if (format == FORMAT_NHWC) return dimension == 'N' ? 0 : dimension == 'H' ? 1 : dimension == 'W' ? 2 : 3;
    return dimension == 'N' ? 0 : dimension == 'C' ? 1 : dimension == 'H' ? 2 : 3;
}
template <typename T> T GetTensorDim(const std::vector<T> &attributes, TensorFormat format, char dimension)
{
    return attributes[std::size_t(DimIndex(format, dimension))];
}
inline int64 GetTensorDim(const Tensor &tensor, TensorFormat format, char dimension) { return tensor.dim_size(DimIndex(format, dimension)); }
inline TensorShape ShapeFromFormat(TensorFormat format, int64 N, int64 H, int64 W, int64 C)
{
    return format == FORMAT_NHWC ? TensorShape({N, H, W, C}) : TensorShape({N, C, H, W});
}
}  // namespace tensorflow
