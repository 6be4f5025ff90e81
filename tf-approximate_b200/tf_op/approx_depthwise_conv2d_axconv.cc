// TensorFlow op-kernel shim for the depthwise variant of the table convolution.  The reference has no such op (its
// launcher rejects grouped shapes, tf2/src/approx_nn_conv_ops.cpp:229-232); this kernel is meant to be registered
// under a new op `ApproxDepthwiseConv2DWithMinMaxVars` whose REGISTER_OP repeats the inputs and attributes of
// `ApproxConv2DWithMinMaxVars` (tf2/src/approx_nn_ops.cpp:38-54) with the filter laid out as TensorFlow's
// DepthwiseConv2dNative does, [KH, KW, C, multiplier].  Same structure as approx_conv2d_axconv.cc.
// Build inside the reference's tree: add this file and the new REGISTER_OP to the plugin's sources, add include/ of
// this repository to the include path and link libaxconv.so.
#include <cuda_runtime_api.h>

#include <string>
#include <vector>

#include "axconv.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/util/padding.h"
#include "tensorflow/core/util/tensor_format.h"

namespace tensorflow {

namespace {

// Status codes of the library carry TensorFlow's numeric error codes for the conditions the reference reports.
Status FromAxc(int st)
{
    switch (st) {
    case AXC_OK: return Status::OK();
    case AXC_INVALID_ARGUMENT: return errors::InvalidArgument("ApproxDepthwiseConv2D: invalid argument");
    case AXC_UNIMPLEMENTED: return errors::Unimplemented("ApproxDepthwiseConv2D: not implemented for these attributes");
    default: return errors::Internal("ApproxDepthwiseConv2D: ", axc_status_string(st), ", cudaError ", axc_last_cuda_error());
    }
}

}  // namespace

class AxconvApproxDepthwiseConv2DOp : public OpKernel {
public:
    explicit AxconvApproxDepthwiseConv2DOp(OpKernelConstruction *ctx) : OpKernel(ctx)
    {
        // attributes as InitApproxConv2DParameters reads them (tf2/src/approx_nn_conv_ops.cpp:254-309) and the
        // table attributes of BaseTableApproxOpType_t (tf2/src/approx_ops_types.h:99-122)
        int num_bits = 0;
        std::string file, format;
        std::vector<int32> strides, dilations;
        OP_REQUIRES_OK(ctx, ctx->GetAttr("num_bits", &num_bits));
        OP_REQUIRES_OK(ctx, ctx->GetAttr("mul_map_file", &file));
        OP_REQUIRES_OK(ctx, ctx->GetAttr("strides", &strides));
        OP_REQUIRES_OK(ctx, ctx->GetAttr("dilations", &dilations));
        OP_REQUIRES_OK(ctx, ctx->GetAttr("padding", &padding_));
        OP_REQUIRES_OK(ctx, ctx->GetAttr("data_format", &format));
        OP_REQUIRES(ctx, FormatFromString(format, &format_), errors::InvalidArgument("Invalid data format"));
        OP_REQUIRES(ctx, strides.size() == 4, errors::InvalidArgument("Sliding window strides field must specify 4 dimensions"));
        OP_REQUIRES(ctx, dilations.size() == 4, errors::InvalidArgument("Sliding window dilations field must specify 4 dimensions"));
        OP_REQUIRES(ctx, GetTensorDim(strides, format_, 'N') == 1 && GetTensorDim(strides, format_, 'C') == 1,
                    errors::InvalidArgument("Current implementation does not yet support strides in the batch and depth dimensions."));
        OP_REQUIRES(ctx, GetTensorDim(dilations, format_, 'N') == 1 && GetTensorDim(dilations, format_, 'C') == 1,
                    errors::InvalidArgument("Current implementation does not yet support dilations in the batch and depth dimensions."));
        stride_h_ = GetTensorDim(strides, format_, 'H');
        stride_w_ = GetTensorDim(strides, format_, 'W');
        dil_h_ = GetTensorDim(dilations, format_, 'H');
        dil_w_ = GetTensorDim(dilations, format_, 'W');
        const int st = axc_table_create_from_file(file.c_str(), num_bits, &table_);
        OP_REQUIRES(ctx, st == AXC_OK, errors::InvalidArgument("ApproxTF: Couldn't read the lookup table!"));
    }

    ~AxconvApproxDepthwiseConv2DOp() override { axc_table_destroy(table_); }

    void Compute(OpKernelContext *ctx) override
    {
        const Tensor &input = ctx->input(0);
        const Tensor &filter = ctx->input(1);
        OP_REQUIRES(ctx, input.dims() == 4, errors::InvalidArgument("input must be 4-dimensional"));
        OP_REQUIRES(ctx, filter.dims() == 4, errors::InvalidArgument("filter must be 4-dimensional"));
        axc_conv_desc d = {};
        d.n = static_cast<int32_t>(GetTensorDim(input, format_, 'N'));
        d.h = static_cast<int32_t>(GetTensorDim(input, format_, 'H'));
        d.w = static_cast<int32_t>(GetTensorDim(input, format_, 'W'));
        d.c = static_cast<int32_t>(GetTensorDim(input, format_, 'C'));
        d.kh = static_cast<int32_t>(filter.dim_size(0));
        d.kw = static_cast<int32_t>(filter.dim_size(1));
        d.filter_c = static_cast<int32_t>(filter.dim_size(2));
        d.cout = static_cast<int32_t>(filter.dim_size(3));      // the channel multiplier
        d.stride_h = stride_h_;
        d.stride_w = stride_w_;
        d.dil_h = dil_h_;
        d.dil_w = dil_w_;
        d.padding = padding_ == SAME ? AXC_PADDING_SAME : padding_ == VALID ? AXC_PADDING_VALID : AXC_PADDING_EXPLICIT;
        d.data_format = format_ == FORMAT_NHWC ? AXC_FORMAT_NHWC : AXC_FORMAT_NCHW;
        int64_t dims[4];
        OP_REQUIRES_OK(ctx, FromAxc(axc_depthwise_conv2d_output_dims(&d, dims)));
        Tensor *output = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, ShapeFromFormat(format_, dims[0], dims[1], dims[2], dims[3]), &output));
        if (output->NumElements() == 0) return;             // as the reference: nothing to do (:449-450)

        // The workspace holds the quantised filter and the filter sums of this call; kept with the op instance so
        // that no allocation happens per call.
        size_t ws_bytes = 0;
        OP_REQUIRES_OK(ctx, FromAxc(axc_depthwise_conv2d_workspace_bytes(&d, &ws_bytes)));
        if (ws_bytes > ws_bytes_) {
            OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_UINT8, TensorShape({static_cast<int64>(ws_bytes)}), &workspace_));
            ws_bytes_ = ws_bytes;
        }
        int device = 0;
        OP_REQUIRES(ctx, cudaGetDevice(&device) == cudaSuccess, errors::Internal("No GPU device is current."));
        cudaStream_t stream = ctx->eigen_device<Eigen::GpuDevice>().stream();
        // inputs 2..5 are host-memory scalars, as in the reference's kernel builder (:691-694)
        const int st = axc_depthwise_conv2d_forward(table_, &d, input.flat<float>().data(), filter.flat<float>().data(),
                                          ctx->input(2).scalar<float>()(), ctx->input(3).scalar<float>()(),
                                          ctx->input(4).scalar<float>()(), ctx->input(5).scalar<float>()(),
                                          output->flat<float>().data(), workspace_.flat<uint8>().data(), ws_bytes_, nullptr,
                                          device, stream);
        OP_REQUIRES_OK(ctx, FromAxc(st));
    }

private:
    axc_table *table_ = nullptr;
    Padding padding_ = SAME;
    TensorFormat format_ = FORMAT_NHWC;
    int stride_h_ = 1, stride_w_ = 1, dil_h_ = 1, dil_w_ = 1;
    Tensor workspace_;
    size_t ws_bytes_ = 0;
};

REGISTER_KERNEL_BUILDER(Name("ApproxDepthwiseConv2DWithMinMaxVars")
                            .Device(DEVICE_GPU)
                            .TypeConstraint<float>("T")
                            .HostMemory("input_min")
                            .HostMemory("input_max")
                            .HostMemory("filter_min")
                            .HostMemory("filter_max"),
                        AxconvApproxDepthwiseConv2DOp);

}  // namespace tensorflow
