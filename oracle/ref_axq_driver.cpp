// TEST INFRASTRUCTURE.  C entry points around the reference's first-generation op, compiled from the reference
// checkout where it lies (tf1/axqconv/axqconv.cc with quantization_utils.h, approximate_selector.h and the
// multiplier sources of tf1/axqconv/axmult) against the stand-in headers of tf1_stub/.  The op's own Compute()
// runs: zero points, the integer functor with its zero-point terms, the output range.
#include "axqconv.cc"

using namespace tensorflow;

// The selector's table for a multiplier name, with or without weight tuning
// (tf1/axqconv/approximate_selector.h:19-84).  out: int32[65536], index = data * 256 + weight.
extern "C" int refq_table(const char *name, int tune, int32_t *out)
{
    try {
        ApproximateSelector sel;
        sel.init(name, tune != 0);
        for (int a = 0; a < 256; ++a)
            for (int b = 0; b < 256; ++b) out[a * 256 + b] = sel.multiplicate(a, b);
    } catch (std::invalid_argument &) {
        return 1;
    }
    return 0;
}

// One Compute() of AxConv2D.  Returns 0, or 1 when the op reported an error.
extern "C" int refq_conv2d(const char *axmult, int tune, const uint8_t *input, int n, int h, int w, int c,
                           const uint8_t *filter, int kh, int kw, int cout, float min_input, float max_input,
                           float min_filter, float max_filter, int stride, int padding_same, int32_t *output,
                           float *min_output, float *max_output)
{
    OpKernelConstruction cons;
    cons.list_attrs["strides"] = {1, stride, stride, 1};
    cons.list_attrs["dilations"] = {1, 1, 1, 1};
    cons.string_attrs["padding"] = padding_same ? "SAME" : "VALID";
    cons.string_attrs["AxMult"] = axmult;
    cons.bool_attrs["AxTune"] = tune != 0;
    AxQuantizedConv2DOp<quint8, quint8, qint32, ReferenceAxConvFunctor> op(&cons);
    if (!cons.status.ok()) return 1;
    OpKernelContext ctx;
    float scalars[4] = {min_input, max_input, min_filter, max_filter};
    ctx.inputs.push_back(Tensor(const_cast<uint8_t *>(input), TensorShape({n, h, w, c})));
    ctx.inputs.push_back(Tensor(const_cast<uint8_t *>(filter), TensorShape({kh, kw, c, cout})));
    for (int i = 0; i < 4; ++i) ctx.inputs.push_back(Tensor(&scalars[i], TensorShape({})));
    ctx.output_buffers = {output, min_output, max_output};
    op.Compute(&ctx);
    return ctx.status.ok() ? 0 : 1;
}
