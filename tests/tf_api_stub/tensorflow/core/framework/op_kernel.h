// TEST INFRASTRUCTURE.  A stand-in for the part of TensorFlow's op-kernel API that the op-kernel shim
// (tf-approximate_b200/tf_op/approx_conv2d_axconv.cc) uses, written for this repository so that the shim can be
// compiled - and its Compute() run on device buffers - where TensorFlow is not installed.  The classes have the
// member functions TensorFlow 2.x gives them, with small inline bodies: tensors are views of (or owners of) CUDA
// device memory, attributes come from a map, kernel registrations go into a list the test harness
// (tests/tf_api_stub/shim_harness.cc) looks the op up in.  Nothing here is TensorFlow code.
#pragma once
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

namespace Eigen {
struct GpuDevice {
    cudaStream_t stream_ = nullptr;
    cudaStream_t stream() const { return stream_; }
};
}  // namespace Eigen

namespace tensorflow {
typedef std::int32_t int32;
typedef std::int64_t int64;
typedef std::uint8_t uint8;

enum DataType { DT_FLOAT = 1, DT_UINT8 = 4 };
static const char *const DEVICE_GPU = "GPU";

class Status {
public:
    Status() {}
    Status(int code, const std::string &msg) : code_(code), msg_(msg) {}
    static Status OK() { return Status(); }
    bool ok() const { return code_ == 0; }
    int code() const { return code_; }
    const std::string &error_message() const { return msg_; }
private:
    int code_ = 0;
    std::string msg_;
};

namespace errors {
namespace detail {
inline void append(std::ostringstream &) {}
template <typename T, typename... Rest> void append(std::ostringstream &os, const T &v, const Rest &... rest)
{
    os << v;
    append(os, rest...);
}
template <typename... Args> Status make(int code, const Args &... args)
{
    std::ostringstream os;
    append(os, args...);
    return Status(code, os.str());
}
}  // namespace detail
// TensorFlow's numeric error codes
template <typename... Args> Status InvalidArgument(Args... args) { return detail::make(3, args...); }
template <typename... Args> Status Unimplemented(Args... args) { return detail::make(12, args...); }
template <typename... Args> Status Internal(Args... args) { return detail::make(13, args...); }
}  // namespace errors

class TensorShape {
public:
    TensorShape() {}
    TensorShape(std::initializer_list<int64> dims) : dims_(dims) {}
    int dims() const { return int(dims_.size()); }
    int64 dim_size(int index) const { return dims_[std::size_t(index)]; }
    int64 num_elements() const
    {
        int64 n = 1;
        for (int64 d : dims_) n *= d;
        return n;
    }
private:
    std::vector<int64> dims_;
};

class Tensor {
public:
    Tensor() {}
    // a view of memory somebody else owns (device memory for tensors, host memory for the scalar inputs)
    Tensor(void *data, const TensorShape &shape) : data_(data), shape_(shape) {}
    // a tensor that owns device memory
    static Tensor OwnDevice(const TensorShape &shape, std::size_t bytes, cudaError_t *err)
    {
        Tensor t;
        void *p = nullptr;
        *err = cudaMalloc(&p, bytes ? bytes : 1);
        if (*err == cudaSuccess) {
            t.owner_ = std::shared_ptr<void>(p, [](void *q) { cudaFree(q); });
            t.data_ = p;
            t.shape_ = shape;
        }
        return t;
    }
    int dims() const { return shape_.dims(); }
    int64 dim_size(int index) const { return shape_.dim_size(index); }
    int64 NumElements() const { return shape_.num_elements(); }
    const TensorShape &shape() const { return shape_; }
    template <typename T> struct FlatView {
        T *ptr;
        T *data() const { return ptr; }
    };
    template <typename T> struct ScalarView {
        const T *ptr;
        T operator()() const { return *ptr; }
    };
    template <typename T> FlatView<T> flat() { return FlatView<T>{static_cast<T *>(data_)}; }
    template <typename T> FlatView<const T> flat() const { return FlatView<const T>{static_cast<const T *>(data_)}; }
    template <typename T> ScalarView<T> scalar() const { return ScalarView<T>{static_cast<const T *>(data_)}; }
private:
    void *data_ = nullptr;
    TensorShape shape_;
    std::shared_ptr<void> owner_;
};

enum Padding { VALID = 1, SAME = 2, EXPLICIT = 3 };

class OpKernelConstruction {
public:
    std::map<std::string, int> int_attrs;
    std::map<std::string, std::string> string_attrs;
    std::map<std::string, std::vector<int32>> list_attrs;
    Status status;
    Status GetAttr(const std::string &name, int *value) const
    {
        auto it = int_attrs.find(name);
        if (it == int_attrs.end()) return errors::InvalidArgument("no attribute ", name);
        *value = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, std::string *value) const
    {
        auto it = string_attrs.find(name);
        if (it == string_attrs.end()) return errors::InvalidArgument("no attribute ", name);
        *value = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, std::vector<int32> *value) const
    {
        auto it = list_attrs.find(name);
        if (it == list_attrs.end()) return errors::InvalidArgument("no attribute ", name);
        *value = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, Padding *value) const
    {
        auto it = string_attrs.find(name);
        if (it == string_attrs.end()) return errors::InvalidArgument("no attribute ", name);
        *value = it->second == "SAME" ? SAME : it->second == "VALID" ? VALID : EXPLICIT;
        return Status::OK();
    }
    void CtxFailure(const Status &s) { if (status.ok()) status = s; }
    void CtxFailureWithWarning(const Status &s) { CtxFailure(s); }
};

class OpKernelContext {
public:
    std::vector<Tensor> inputs;
    std::map<int, void *> output_buffers;     // device memory the harness wants output i written to
    std::map<int, Tensor> outputs;
    Eigen::GpuDevice gpu;
    Status status;
    const Tensor &input(int index) { return inputs[std::size_t(index)]; }
    Status allocate_output(int index, const TensorShape &shape, Tensor **tensor)
    {
        auto it = output_buffers.find(index);
        if (it == output_buffers.end()) return errors::Internal("no buffer for output ", index);
        outputs[index] = Tensor(it->second, shape);
        *tensor = &outputs[index];
        return Status::OK();
    }
    Status allocate_temp(DataType type, const TensorShape &shape, Tensor *out_temp)
    {
        cudaError_t err = cudaSuccess;
        *out_temp = Tensor::OwnDevice(shape, std::size_t(shape.num_elements()) * (type == DT_FLOAT ? 4 : 1), &err);
        return err == cudaSuccess ? Status::OK() : errors::Internal("device allocation failed: ", cudaGetErrorString(err));
    }
    template <typename Device> const Device &eigen_device() const;
    void CtxFailure(const Status &s) { if (status.ok()) status = s; }
    void CtxFailureWithWarning(const Status &s) { CtxFailure(s); }
};
template <> inline const Eigen::GpuDevice &OpKernelContext::eigen_device<Eigen::GpuDevice>() const { return gpu; }

class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction *) {}
    virtual ~OpKernel() {}
    virtual void Compute(OpKernelContext *ctx) = 0;
};

class KernelDefBuilder {
public:
    explicit KernelDefBuilder(const char *op_name) : op_name_(op_name) {}
    KernelDefBuilder &Device(const char *device_type) { device_ = device_type; return *this; }
    template <typename T> KernelDefBuilder &TypeConstraint(const char *) { return *this; }
    KernelDefBuilder &HostMemory(const char *arg_name) { host_memory_.push_back(arg_name); return *this; }
    const std::string &op_name() const { return op_name_; }
    const std::string &device() const { return device_; }
    const std::vector<std::string> &host_memory() const { return host_memory_; }
private:
    std::string op_name_, device_;
    std::vector<std::string> host_memory_;
};
typedef KernelDefBuilder Name;

namespace kernel_factory {
struct Registration {
    KernelDefBuilder def;
    OpKernel *(*create)(OpKernelConstruction *);
};
inline std::vector<Registration> &registry()
{
    static std::vector<Registration> r;
    return r;
}
struct OpKernelRegistrar {
    OpKernelRegistrar(const KernelDefBuilder &def, OpKernel *(*create)(OpKernelConstruction *)) { registry().push_back(Registration{def, create}); }
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
