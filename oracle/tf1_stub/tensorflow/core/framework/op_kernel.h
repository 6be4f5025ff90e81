// TEST INFRASTRUCTURE.  Minimal stand-in for the TensorFlow 1.x op-kernel API, just wide enough to compile the
// reference's first-generation op (tf1/axqconv/axqconv.cc with quantization_utils.h and approximate_selector.h)
// where it lies, without TensorFlow or Eigen, and to run its Compute() on host arrays.  Written for this build;
// nothing here is TensorFlow code.  Only what those files touch is provided; Eigen expressions that the header
// uses in functions nobody calls are swallowed by `AnyExpr`.
#pragma once
#include <array>
#include <cassert>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <initializer_list>
#include <iostream>
#include <limits>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace Eigen {
typedef long DenseIndex;
struct ThreadPoolDevice {};
template <typename T, std::size_t N> using array = std::array<T, N>;
struct QInt32;
struct QUInt8 {
    QUInt8() : value(0) {}
    QUInt8(const std::uint8_t v) : value(v) {}
    operator int() const { return static_cast<int>(value); }
    std::uint8_t value;
};
struct QInt8 {
    QInt8() : value(0) {}
    QInt8(const std::int8_t v) : value(v) {}
    operator int() const { return static_cast<int>(value); }
    std::int8_t value;
};
struct QUInt16 {
    QUInt16() : value(0) {}
    QUInt16(const std::uint16_t v) : value(v) {}
    operator int() const { return static_cast<int>(value); }
    std::uint16_t value;
};
struct QInt16 {
    QInt16() : value(0) {}
    QInt16(const std::int16_t v) : value(v) {}
    operator int() const { return static_cast<int>(value); }
    std::int16_t value;
};
struct QInt32 {
    QInt32() : value(0) {}
    QInt32(const std::int32_t v) : value(v) {}
    operator int() const { return static_cast<int>(value); }
    std::int32_t value;
};
template <typename T> struct NumTraits {
    static T lowest() { return std::numeric_limits<T>::lowest(); }
    static T highest() { return std::numeric_limits<T>::max(); }
};
template <> struct NumTraits<QUInt8> { static QUInt8 lowest() { return QUInt8(0); } static QUInt8 highest() { return QUInt8(255); } };
template <> struct NumTraits<QInt8> { static QInt8 lowest() { return QInt8(-128); } static QInt8 highest() { return QInt8(127); } };
template <> struct NumTraits<QUInt16> { static QUInt16 lowest() { return QUInt16(0); } static QUInt16 highest() { return QUInt16(65535); } };
template <> struct NumTraits<QInt16> { static QInt16 lowest() { return QInt16(-32768); } static QInt16 highest() { return QInt16(32767); } };
template <> struct NumTraits<QInt32> {
    static QInt32 lowest() { return QInt32(std::numeric_limits<std::int32_t>::min()); }
    static QInt32 highest() { return QInt32(std::numeric_limits<std::int32_t>::max()); }
};
namespace numext {
template <typename T> T mini(const T &a, const T &b) { return b < a ? b : a; }
template <typename T> T maxi(const T &a, const T &b) { return a < b ? b : a; }
}  // namespace numext
}  // namespace Eigen

#define EIGEN_ALWAYS_INLINE inline
#define EIGEN_STRONG_INLINE inline
#define EIGEN_DEVICE_FUNC
#define EIGEN_EMPTY_STRUCT_CTOR(X)

namespace tensorflow {
typedef std::uint8_t uint8;
typedef std::uint16_t uint16;
typedef std::uint32_t uint32;
typedef std::uint64_t uint64;
typedef std::int8_t int8;
typedef std::int16_t int16;
typedef std::int32_t int32;
typedef std::int64_t int64;
typedef Eigen::QUInt8 quint8;
typedef Eigen::QInt8 qint8;
typedef Eigen::QUInt16 quint16;
typedef Eigen::QInt16 qint16;
typedef Eigen::QInt32 qint32;
using std::string;

enum DataType { DT_INVALID = 0, DT_FLOAT, DT_QUINT8, DT_QINT8, DT_QUINT16, DT_QINT16, DT_QINT32, DT_INT32 };
template <typename T> struct DataTypeToEnum { static DataType v() { return DT_INVALID; } };
enum Padding { VALID = 1, SAME = 2 };
static const char *const DEVICE_CPU = "CPU";

class Status {
public:
    Status() : m_ok(true) {}
    explicit Status(const std::string &msg) : m_ok(false), m_msg(msg) {}
    static Status OK() { return Status(); }
    bool ok() const { return m_ok; }
    const std::string &error_message() const { return m_msg; }
private:
    bool m_ok;
    std::string m_msg;
};

namespace errors {
template <typename... Args> Status InvalidArgument(const char *msg, Args...) { return Status(msg); }
template <typename... Args> Status Unimplemented(const char *msg, Args...) { return Status(msg); }
template <typename... Args> Status Internal(const char *msg, Args...) { return Status(msg); }
}  // namespace errors

// Swallows any Eigen expression the header builds in functions that are never called here.
struct AnyExpr {
    AnyExpr() {}
    template <typename T> AnyExpr(const T &) {}
    template <typename T> AnyExpr cast() const { return AnyExpr(); }
    template <typename F> AnyExpr unaryExpr(const F &) const { return AnyExpr(); }
    template <typename T> AnyExpr cwiseMax(const T &) const { return AnyExpr(); }
    template <typename T> AnyExpr cwiseMin(const T &) const { return AnyExpr(); }
    template <typename T> AnyExpr reshape(const T &) const { return AnyExpr(); }
    template <typename T> AnyExpr broadcast(const T &) const { return AnyExpr(); }
    AnyExpr round() const { return AnyExpr(); }
    template <typename D> AnyExpr &device(const D &) { return *this; }
    long size() const { return 0; }
};
template <typename T> AnyExpr operator*(const AnyExpr &, const T &) { return AnyExpr(); }
template <typename T> AnyExpr operator+(const AnyExpr &, const T &) { return AnyExpr(); }
template <typename T> AnyExpr operator-(const AnyExpr &, const T &) { return AnyExpr(); }
template <typename T> AnyExpr operator/(const AnyExpr &, const T &) { return AnyExpr(); }

// What Tensor::flat<T>() returns: element access for the code that runs, AnyExpr for the code that does not.
template <typename T> struct Flat : AnyExpr {
    T *m_data;
    long m_size;
    Flat(T *d, long n) : m_data(d), m_size(n) {}
    T &operator()(long i) const { return m_data[i]; }
    T *data() const { return m_data; }
    long size() const { return m_size; }
    template <typename D> Flat &device(const D &) { return *this; }
    Flat &operator=(const AnyExpr &) { return *this; }
};

class TensorShape {
public:
    TensorShape() {}
    TensorShape(std::initializer_list<int64> d) : m_dims(d) {}
    int dims() const { return int(m_dims.size()); }
    int64 dim_size(int i) const { return m_dims[std::size_t(i)]; }
    int64 num_elements() const { int64 n = 1; for (int64 v : m_dims) n *= v; return n; }
    std::string DebugString() const { return "[shape]"; }
private:
    std::vector<int64> m_dims;
};

// A view of host memory (the driver owns the bytes) or, when default-made by allocate_output, a small owning buffer.
class Tensor {
public:
    Tensor() : m_ptr(nullptr) {}
    Tensor(DataType, const TensorShape &s) : m_shape(s), m_ptr(nullptr) {}
    Tensor(void *p, const TensorShape &s) : m_shape(s), m_ptr(p) {}
    int dims() const { return m_shape.dims(); }
    int64 dim_size(int i) const { return m_shape.dim_size(i); }
    int64 NumElements() const { return m_shape.num_elements(); }
    const TensorShape &shape() const { return m_shape; }
    DataType dtype() const { return DT_INVALID; }
    template <typename T> Flat<T> flat() { return Flat<T>(static_cast<T *>(m_ptr), long(NumElements())); }
    template <typename T> Flat<const T> flat() const { return Flat<const T>(static_cast<const T *>(m_ptr), long(NumElements())); }
    void *raw() const { return m_ptr; }
private:
    TensorShape m_shape;
    void *m_ptr;
};

// Attribute bag standing in for OpKernelConstruction.
class OpKernelConstruction {
public:
    std::map<std::string, std::vector<int32>> list_attrs;
    std::map<std::string, std::string> string_attrs;
    std::map<std::string, bool> bool_attrs;
    Status status;
    Status GetAttr(const std::string &name, std::vector<int32> *v) const {
        auto it = list_attrs.find(name);
        if (it == list_attrs.end()) return Status("missing attr " + name);
        *v = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, std::string *v) const {
        auto it = string_attrs.find(name);
        if (it == string_attrs.end()) return Status("missing attr " + name);
        *v = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, bool *v) const {
        auto it = bool_attrs.find(name);
        if (it == bool_attrs.end()) return Status("missing attr " + name);
        *v = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, Padding *v) const {
        auto it = string_attrs.find(name);
        if (it == string_attrs.end()) return Status("missing attr " + name);
        *v = it->second == "VALID" ? VALID : SAME;
        return Status::OK();
    }
    void SetStatus(const Status &s) { if (status.ok()) status = s; }
    void CtxFailure(const Status &s) { SetStatus(s); }
};

// Inputs are views set by the driver; outputs are written into buffers the driver registered per index.
class OpKernelContext {
public:
    std::vector<Tensor> inputs;
    std::vector<void *> output_buffers;       // where output i goes
    std::vector<Tensor> outputs;
    Status status;
    const Tensor &input(int i) const { return inputs[std::size_t(i)]; }
    Status allocate_output(int i, const TensorShape &shape, Tensor **out) {
        if (outputs.size() <= std::size_t(i)) outputs.resize(std::size_t(i) + 1);
        outputs[std::size_t(i)] = Tensor(output_buffers[std::size_t(i)], shape);
        *out = &outputs[std::size_t(i)];
        return Status::OK();
    }
    void SetStatus(const Status &s) { if (status.ok()) status = s; }
    void CtxFailure(const Status &s) { SetStatus(s); }
};

class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction *) {}
    virtual ~OpKernel() {}
    virtual void Compute(OpKernelContext *context) = 0;
};

// SAME / VALID output size of one dimension, dilation 1: the published TensorFlow rule.
inline Status GetWindowedOutputSize(int64 input_size, int64 filter_size, int64 stride, Padding padding, int64 *output_size,
                                    int64 *padding_size)
{
    if (stride <= 0) return Status("stride must be > 0");
    if (padding == VALID) {
        *output_size = (input_size - filter_size + stride) / stride;
        *padding_size = 0;
    } else {
        *output_size = (input_size + stride - 1) / stride;
        const int64 needed = (*output_size - 1) * stride + filter_size - input_size;
        *padding_size = needed > 0 ? needed / 2 : 0;
    }
    if (*output_size < 0) return Status("computed output size would be negative");
    return Status::OK();
}

// Op and kernel registration: parsed, not recorded.
namespace shape_inference {
struct DimensionHandle {};
struct ShapeHandle {};
struct InferenceContext {
    ShapeHandle input(int) { return ShapeHandle(); }
    Status WithRank(ShapeHandle, int, ShapeHandle *) { return Status::OK(); }
    ShapeHandle Scalar() { return ShapeHandle(); }
    void set_output(int, ShapeHandle) {}
};
inline Status Conv2DShape(InferenceContext *) { return Status::OK(); }
}  // namespace shape_inference
struct OpDefBuilderStub {
    OpDefBuilderStub &Input(const char *) { return *this; }
    OpDefBuilderStub &Output(const char *) { return *this; }
    OpDefBuilderStub &Attr(const char *) { return *this; }
    template <typename F> OpDefBuilderStub &SetShapeFn(F) { return *this; }
};
struct KernelDefBuilderStub {
    KernelDefBuilderStub &Device(const char *) { return *this; }
    template <typename T> KernelDefBuilderStub &TypeConstraint(const char *) { return *this; }
};
inline KernelDefBuilderStub Name(const char *) { return KernelDefBuilderStub(); }
}  // namespace tensorflow

#define AXSTUB_CAT2(a, b) a##b
#define AXSTUB_CAT(a, b) AXSTUB_CAT2(a, b)
#define REGISTER_OP(name) static ::tensorflow::OpDefBuilderStub AXSTUB_CAT(axstub_op_, __LINE__) = ::tensorflow::OpDefBuilderStub()
// instantiates the kernel class so that it is compiled; the driver constructs it directly
#define REGISTER_KERNEL_BUILDER(builder, ...) typedef __VA_ARGS__ AXSTUB_CAT(AxStubRegisteredKernel, __LINE__)
#define TF_RETURN_IF_ERROR(...)                          \
    do {                                                 \
        ::tensorflow::Status _s(__VA_ARGS__);            \
        if (!_s.ok()) return _s;                         \
    } while (0)
#define TF_PREDICT_TRUE(x) (x)
#define TF_PREDICT_FALSE(x) (x)
#define TF_DISALLOW_COPY_AND_ASSIGN(T)
#define OP_REQUIRES_OK(CTX, ...)                         \
    do {                                                 \
        ::tensorflow::Status _s(__VA_ARGS__);            \
        if (!_s.ok()) { (CTX)->CtxFailure(_s); return; } \
    } while (0)
#define OP_REQUIRES(CTX, EXP, STATUS)                    \
    do {                                                 \
        if (!(EXP)) { (CTX)->CtxFailure(STATUS); return; } \
    } while (0)
#define CHECK(x) assert(x)
#define CHECK_GT(a, b) assert((a) > (b))
#define DCHECK(x) assert(x)
#define DCHECK_EQ(a, b) assert((a) == (b))
#define DCHECK_GE(a, b) assert((a) >= (b))
#define DCHECK_LE(a, b) assert((a) <= (b))
#define LOG(x) if (true) {} else std::cerr
#define VLOG(n) if (true) {} else std::cerr
