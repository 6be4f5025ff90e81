// TEST INFRASTRUCTURE.  A stand-in for the part of TensorFlow's op-kernel API that the op-kernel shim
// (tf-approximate_b200/tf_op/approx_conv2d_axconv.cc) uses, written for this repository so that the shim can be
// compiled where TensorFlow is not installed.  Declarations only, with the signatures TensorFlow 2.x gives them;
// nothing here is TensorFlow code and nothing here runs.
#pragma once
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

namespace Eigen {
struct GpuDevice {
    cudaStream_t stream() const;
};
}  // namespace Eigen

namespace tensorflow {
typedef std::int32_t int32;
typedef std::int64_t int64;
typedef std::uint8_t uint8;

enum DataType { DT_FLOAT = 1, DT_UINT8 = 4 };
extern const char *const DEVICE_GPU;

class Status {
public:
    static Status OK();
    bool ok() const;
};

namespace errors {
template <typename... Args> Status InvalidArgument(Args...);
template <typename... Args> Status Unimplemented(Args...);
template <typename... Args> Status Internal(Args...);
}  // namespace errors

class TensorShape {
public:
    TensorShape();
    TensorShape(std::initializer_list<int64> dims);
};

class Tensor {
public:
    Tensor();
    int dims() const;
    int64 dim_size(int index) const;
    int64 NumElements() const;
    template <typename T> struct FlatView {
        T *data() const;
    };
    template <typename T> struct ScalarView {
        T operator()() const;
    };
    template <typename T> FlatView<T> flat();
    template <typename T> FlatView<const T> flat() const;
    template <typename T> ScalarView<T> scalar() const;
};

enum Padding { VALID = 1, SAME = 2, EXPLICIT = 3 };

class OpKernelConstruction {
public:
    Status GetAttr(const std::string &name, int *value) const;
    Status GetAttr(const std::string &name, std::string *value) const;
    Status GetAttr(const std::string &name, std::vector<int32> *value) const;
    Status GetAttr(const std::string &name, Padding *value) const;
    void CtxFailure(const Status &s);
    void CtxFailureWithWarning(const Status &s);
};

class OpKernelContext {
public:
    const Tensor &input(int index);
    Status allocate_output(int index, const TensorShape &shape, Tensor **tensor);
    Status allocate_temp(DataType type, const TensorShape &shape, Tensor *out_temp);
    template <typename Device> const Device &eigen_device() const;
    void CtxFailure(const Status &s);
    void CtxFailureWithWarning(const Status &s);
};

class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction *ctx);
    virtual ~OpKernel();
    virtual void Compute(OpKernelContext *ctx) = 0;
};

class KernelDefBuilder {
public:
    explicit KernelDefBuilder(const char *op_name);
    KernelDefBuilder &Device(const char *device_type);
    template <typename T> KernelDefBuilder &TypeConstraint(const char *attr_name);
    KernelDefBuilder &HostMemory(const char *arg_name);
};
typedef KernelDefBuilder Name;

namespace kernel_factory {
struct OpKernelRegistrar {
    OpKernelRegistrar(const KernelDefBuilder &def, OpKernel *(*create)(OpKernelConstruction *));
};
}  // namespace kernel_factory
}  // namespace tensorflow

#define OP_REQUIRES(CTX, EXP, STATUS)     \
    do {                                  \
        if (!(EXP)) {                     \
            (CTX)->CtxFailure((STATUS));  \
            return;                       \
        }                                 \
    } while (0)
#define OP_REQUIRES_OK(CTX, ...)                         \
    do {                                                 \
        ::tensorflow::Status _s(__VA_ARGS__);            \
        if (!_s.ok()) {                                  \
            (CTX)->CtxFailureWithWarning(_s);            \
            return;                                      \
        }                                                \
    } while (0)
#define AXC_STUB_CONCAT2(a, b) a##b
#define AXC_STUB_CONCAT(a, b) AXC_STUB_CONCAT2(a, b)
#define REGISTER_KERNEL_BUILDER(kernel_builder, ...)                                                               \
    static ::tensorflow::kernel_factory::OpKernelRegistrar AXC_STUB_CONCAT(registrar__, __LINE__)(                 \
        ::tensorflow::kernel_builder,                                                                              \
        [](::tensorflow::OpKernelConstruction *context) -> ::tensorflow::OpKernel * { return new __VA_ARGS__(context); })
