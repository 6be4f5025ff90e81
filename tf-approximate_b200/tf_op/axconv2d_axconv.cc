// TensorFlow op-kernel shim for the reference's first-generation op `AxConv2D` (quantised uint8 operands in, int32 sums
// and the output range out), re-pointed at libaxconv.  It replaces the kernel class AxQuantizedConv2DOp and its
// functor (tf1/axqconv/axqconv.cc:132-263, 297-451) and nothing else: the op registration (:66-94), the attribute
// names and the multiplier sources (tf1/axqconv/axmult/*.c with the generated axmult.h) stay as they are.
// The op is registered for DEVICE_CPU in the reference, so its tensors live in host memory: this kernel keeps device
// buffers of its own (grown on demand), copies the operands in and the int32 result out on one stream.
// Build inside the reference's tree in place of the kernel registration of axqconv.cc: add include/ of this
// repository to the include path and link libaxconv.so and the CUDA runtime.
#include <cuda_runtime_api.h>

#include <string>
#include <vector>

#include "axconv.h"
#include "axmult.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/util/padding.h"

namespace tensorflow {

class AxconvAxConv2DOp : public OpKernel {
public:
    explicit AxconvAxConv2DOp(OpKernelConstruction *context) : OpKernel(context)
    {
        // the attribute checks of AxQuantizedConv2DOp's constructor (tf1/axqconv/axqconv.cc:301-340), same texts
        std::vector<int32> dilations;
        std::string axmult;
        bool axtune = true;
        OP_REQUIRES_OK(context, context->GetAttr("strides", &strides_));
        OP_REQUIRES(context, strides_.size() == 4, errors::InvalidArgument("Sliding window strides field must specify 4 dimensions"));
        OP_REQUIRES(context, strides_[1] == strides_[2],
                    errors::InvalidArgument("Current implementation only supports equal length strides in the row and column dimensions."));
        OP_REQUIRES(context, (strides_[0] == 1 && strides_[3] == 1),
                    errors::InvalidArgument("Current implementation does not yet support strides in the batch and depth dimensions."));
        OP_REQUIRES_OK(context, context->GetAttr("dilations", &dilations));
        OP_REQUIRES(context, dilations.size() == 4, errors::InvalidArgument("Dilations field must specify 4 dimensions"));
        OP_REQUIRES(context, dilations[1] == 1 && dilations[2] == 1,
                    errors::InvalidArgument("Current implementation only supports dilated rate as 1 in the row and column dimensions."));
        OP_REQUIRES(context, (dilations[0] == 1 && dilations[3] == 1),
                    errors::InvalidArgument("Current implementation does not yet support dilations in the batch and depth dimensions."));
        OP_REQUIRES_OK(context, context->GetAttr("padding", &padding_));
        OP_REQUIRES_OK(context, context->GetAttr("AxMult", &axmult));
        OP_REQUIRES_OK(context, context->GetAttr("AxTune", &axtune));

        // the table of the named multiplier, index = data * 256 + weight (tf1/axqconv/approximate_selector.h:19-44),
        // then the weight tuning (:46-78)
        const int mulid = AxFindId(axmult.c_str());
        OP_REQUIRES(context, mulid >= 0, errors::InvalidArgument("Unknown multiplier \"", axmult, "\""));
        std::vector<uint16_t> lut(65536);
        for (unsigned a = 0; a < 256; ++a)
            for (unsigned b = 0; b < 256; ++b) {
                const unsigned v = AxDo(mulid, a, b);
                OP_REQUIRES(context, v <= 65535u, errors::InvalidArgument("multiplier result does not fit 16 bits"));
                lut[a * 256 + b] = static_cast<uint16_t>(v);
            }
        if (axtune) OP_REQUIRES(context, axc_table_tune_weights(lut.data(), lut.data()) == AXC_OK, errors::Internal("table tuning failed"));
        OP_REQUIRES(context, axc_table_create_from_memory(lut.data(), &table_) == AXC_OK, errors::Internal("table creation failed"));
        OP_REQUIRES(context, cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) == cudaSuccess,
                    errors::Internal("No GPU stream available."));
    }

    ~AxconvAxConv2DOp() override
    {
        for (Buffer *b : {&in_, &filter_, &out_, &ws_}) cudaFree(b->ptr);
        if (stream_) cudaStreamDestroy(stream_);
        axc_table_destroy(table_);
    }

    void Compute(OpKernelContext *context) override
    {
        const Tensor &input = context->input(0);
        const Tensor &filter = context->input(1);
        OP_REQUIRES(context, input.dims() == 4, errors::InvalidArgument("input must be 4-dimensional"));
        OP_REQUIRES(context, filter.dims() == 4, errors::InvalidArgument("filter must be 4-dimensional: "));
        const float min_input = context->input(2).flat<float>()(0);
        const float max_input = context->input(3).flat<float>()(0);
        const float min_filter = context->input(4).flat<float>()(0);
        const float max_filter = context->input(5).flat<float>()(0);
        OP_REQUIRES(context, input.dim_size(3) == filter.dim_size(2),
                    errors::InvalidArgument("input and filter must have the same depth: ", input.dim_size(3), " vs ", filter.dim_size(2)));

        axc_conv_desc d = {};
        d.n = static_cast<int32_t>(input.dim_size(0));
        d.h = static_cast<int32_t>(input.dim_size(1));
        d.w = static_cast<int32_t>(input.dim_size(2));
        d.c = static_cast<int32_t>(input.dim_size(3));
        d.kh = static_cast<int32_t>(filter.dim_size(0));
        d.kw = static_cast<int32_t>(filter.dim_size(1));
        d.filter_c = static_cast<int32_t>(filter.dim_size(2));
        d.cout = static_cast<int32_t>(filter.dim_size(3));
        d.stride_h = d.stride_w = strides_[1];
        d.dil_h = d.dil_w = 1;
        d.padding = padding_ == SAME ? AXC_PADDING_SAME : AXC_PADDING_VALID;
        d.data_format = AXC_FORMAT_NHWC;
        int64_t dims[4];
        OP_REQUIRES(context, axc_conv2d_output_dims(&d, dims) == AXC_OK, errors::InvalidArgument("AxConv2D: invalid shapes"));
        Tensor *output = nullptr;
        OP_REQUIRES_OK(context, context->allocate_output(0, TensorShape({dims[0], dims[1], dims[2], dims[3]}), &output));

        int32_t offset_input = 0, offset_filter = 0;          // FloatToQuantizedUnclamped<T>(0.0f, ...), :365-368
        axc_quantized_zero_point(min_input, max_input, &offset_input);
        axc_quantized_zero_point(min_filter, max_filter, &offset_filter);
        const size_t n_in = static_cast<size_t>(input.NumElements()), n_f = static_cast<size_t>(filter.NumElements());
        const size_t n_out = static_cast<size_t>(output->NumElements());
        if (n_out != 0) {
            size_t ws_bytes = 0;
            OP_REQUIRES(context, axc_qconv2d_workspace_bytes(&d, &ws_bytes) == AXC_OK, errors::InvalidArgument("AxConv2D: invalid shapes"));
            int device = 0;
            OP_REQUIRES(context, cudaGetDevice(&device) == cudaSuccess, errors::Internal("No GPU device is current."));
            OP_REQUIRES(context, in_.reserve(n_in) && filter_.reserve(n_f) && out_.reserve(n_out * 4) && ws_.reserve(ws_bytes),
                        errors::Internal("AxConv2D: device allocation failed"));
            cudaMemcpyAsync(in_.ptr, input.flat<quint8>().data(), n_in, cudaMemcpyHostToDevice, stream_);
            cudaMemcpyAsync(filter_.ptr, filter.flat<quint8>().data(), n_f, cudaMemcpyHostToDevice, stream_);
            const int st = axc_qconv2d_forward(table_, &d, static_cast<const uint8_t *>(in_.ptr), static_cast<const uint8_t *>(filter_.ptr),
                                               offset_input, offset_filter, static_cast<int32_t *>(out_.ptr), ws_.ptr, ws_.bytes, device,
                                               stream_);
            OP_REQUIRES(context, st == AXC_OK,
                        st == AXC_UNIMPLEMENTED ? errors::Unimplemented("AxConv2D: window placement not supported for this stride")
                                                : errors::InvalidArgument("AxConv2D: ", axc_status_string(st)));
            cudaMemcpyAsync(output->flat<qint32>().data(), out_.ptr, n_out * 4, cudaMemcpyDeviceToHost, stream_);
            OP_REQUIRES(context, cudaStreamSynchronize(stream_) == cudaSuccess, errors::Internal("AxConv2D: CUDA error"));
        }

        float range[2] = {0.0f, 0.0f};                        // QuantizationRangeForMultiplication, :429-441
        axc_quantized_output_range(min_input, max_input, min_filter, max_filter, range);
        Tensor *output_min = nullptr;
        OP_REQUIRES_OK(context, context->allocate_output(1, {}, &output_min));
        output_min->flat<float>()(0) = range[0];
        Tensor *output_max = nullptr;
        OP_REQUIRES_OK(context, context->allocate_output(2, {}, &output_max));
        output_max->flat<float>()(0) = range[1];
    }

private:
    struct Buffer {
        void *ptr = nullptr;
        size_t bytes = 0;
        bool reserve(size_t want)
        {
            if (want <= bytes) return true;
            cudaFree(ptr);
            ptr = nullptr;
            bytes = 0;
            if (cudaMalloc(&ptr, want) != cudaSuccess) return false;
            bytes = want;
            return true;
        }
    };
    std::vector<int32> strides_;
    Padding padding_ = SAME;
    axc_table *table_ = nullptr;
    cudaStream_t stream_ = nullptr;
    Buffer in_, filter_, out_, ws_;
};

REGISTER_KERNEL_BUILDER(Name("AxConv2D")
                            .Device(DEVICE_CPU)
                            .TypeConstraint<quint8>("Tinput")
                            .TypeConstraint<quint8>("Tfilter")
                            .TypeConstraint<qint32>("out_type"),
                        AxconvAxConv2DOp);

}  // namespace tensorflow
