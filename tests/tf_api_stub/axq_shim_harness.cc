// TEST INFRASTRUCTURE.  C entry point that runs one Compute() of the first-generation op's shim
// (tf-approximate_b200/tf_op/axconv2d_axconv.cc) on host arrays, with the same signature as the entry point around
// the reference's own op (oracle/ref_axq_driver.cpp), so that a test can put one in the place of the other.
// Compiled against the stand-in headers of oracle/tf1_stub/ and the multiplier header in oracle/_ref/.
#include "axconv2d_axconv.cc"

using namespace tensorflow;

extern "C" int shimq_conv2d(const char *axmult, int tune, const uint8_t *input, int n, int h, int w, int c, const uint8_t *filter,
                            int kh, int kw, int cout, float min_input, float max_input, float min_filter, float max_filter,
                            int stride, int padding_same, int32_t *output, float *min_output, float *max_output)
{
    OpKernelConstruction cons;
    cons.list_attrs["strides"] = {1, stride, stride, 1};
    cons.list_attrs["dilations"] = {1, 1, 1, 1};
    cons.string_attrs["padding"] = padding_same ? "SAME" : "VALID";
    cons.string_attrs["AxMult"] = axmult;
    cons.bool_attrs["AxTune"] = tune != 0;
    AxconvAxConv2DOp op(&cons);
    if (!cons.status.ok()) return 1;
    OpKernelContext ctx;
    float scalars[4] = {min_input, max_input, min_filter, max_filter};
    ctx.inputs.push_back(Tensor(const_cast<uint8_t *>(input), TensorShape({n, h, w, c})));
    ctx.inputs.push_back(Tensor(const_cast<uint8_t *>(filter), TensorShape({kh, kw, c, cout})));
    for (int i = 0; i < 4; ++i) ctx.inputs.push_back(Tensor(&scalars[i], TensorShape({})));
    ctx.output_buffers = {output, min_output, max_output};
    op.Compute(&ctx);
    return ctx.status.ok() ? 0 : 2;
}
