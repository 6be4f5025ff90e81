// TEST INFRASTRUCTURE.  C entry points that drive the op-kernel shim the way TensorFlow's executor would: look the
// kernel up by op name in the registrations the shim's REGISTER_KERNEL_BUILDER made, construct it from attributes,
// and call Compute() with inputs 0, 1 in device memory and inputs 2..5 in host memory (the registration's HostMemory
// pins).  Linked with the shim, libaxconv.so and the CUDA runtime into a test-only library.
#include <cstring>
#include <string>

#include "tensorflow/core/framework/op_kernel.h"

using namespace tensorflow;

namespace {
void put(char *dst, int len, const std::string &s)
{
    if (dst && len > 0) {
        std::strncpy(dst, s.c_str(), std::size_t(len) - 1);
        dst[len - 1] = 0;
    }
}
}  // namespace

// Number of kernels registered for `op_name`; `device` and the comma-separated HostMemory arguments of the first one.
extern "C" int shimtest_registration(const char *op_name, char *device, int device_len, char *host_memory, int host_len)
{
    int n = 0;
    for (const auto &r : kernel_factory::registry()) {
        if (r.def.op_name() != op_name) continue;
        if (n++ == 0) {
            put(device, device_len, r.def.device());
            std::string hm;
            for (const auto &a : r.def.host_memory()) hm += (hm.empty() ? "" : ",") + a;
            put(host_memory, host_len, hm);
        }
    }
    return n;
}

// Constructs the kernel.  Returns NULL and the status (TensorFlow error code, message) when the constructor failed.
extern "C" void *shimtest_create(const char *op_name, const char *mul_map_file, int num_bits, const int *strides4,
                                 const int *dilations4, const char *padding, const char *data_format, int *code, char *msg,
                                 int msg_len)
{
    OpKernelConstruction cons;
    cons.int_attrs["num_bits"] = num_bits;
    cons.string_attrs["mul_map_file"] = mul_map_file;
    cons.string_attrs["padding"] = padding;
    cons.string_attrs["data_format"] = data_format;
    cons.list_attrs["strides"] = {strides4[0], strides4[1], strides4[2], strides4[3]};
    cons.list_attrs["dilations"] = {dilations4[0], dilations4[1], dilations4[2], dilations4[3]};
    cons.list_attrs["explicit_paddings"] = {};
    OpKernel *op = nullptr;
    for (const auto &r : kernel_factory::registry())
        if (r.def.op_name() == op_name) { op = r.create(&cons); break; }
    *code = op ? cons.status.code() : 13;
    put(msg, msg_len, op ? cons.status.error_message() : std::string("no kernel registered for ") + op_name);
    if (op && !cons.status.ok()) { delete op; op = nullptr; }
    return op;
}

extern "C" void shimtest_destroy(void *op) { delete static_cast<OpKernel *>(op); }

// One Compute().  input/filter/output are device pointers, the four ranges host floats; out_dims receives the shape of
// output 0 as the kernel allocated it.  Returns the TensorFlow error code of the context (0 = OK).
extern "C" int shimtest_compute(void *op, float *input, const long long *in_dims, float *filter, const long long *f_dims,
                                const float *ranges4, float *output, long long *out_dims, void *stream, char *msg, int msg_len)
{
    OpKernelContext ctx;
    ctx.gpu.stream_ = static_cast<cudaStream_t>(stream);
    float host[4] = {ranges4[0], ranges4[1], ranges4[2], ranges4[3]};
    ctx.inputs.push_back(Tensor(input, TensorShape({in_dims[0], in_dims[1], in_dims[2], in_dims[3]})));
    ctx.inputs.push_back(Tensor(filter, TensorShape({f_dims[0], f_dims[1], f_dims[2], f_dims[3]})));
    for (int i = 0; i < 4; ++i) ctx.inputs.push_back(Tensor(&host[i], TensorShape()));
    ctx.output_buffers[0] = output;
    static_cast<OpKernel *>(op)->Compute(&ctx);
    auto it = ctx.outputs.find(0);
    for (int i = 0; i < 4; ++i) out_dims[i] = it != ctx.outputs.end() && it->second.dims() == 4 ? it->second.dim_size(i) : -1;
    put(msg, msg_len, ctx.status.error_message());
    return ctx.status.code();
}
