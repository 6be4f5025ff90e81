// TEST INFRASTRUCTURE.  Minimal stand-in for the TensorFlow op-kernel API, just
// wide enough to compile the reference's CPU kernel translation unit
// (tf2/src/approx_nn_conv_kernels.cpp with tf2/src/approx_ops_types.h) where it
// lies, without TensorFlow or Eigen.  Written for this build; nothing here is
// TensorFlow code.  Only what those two files touch is provided.
#pragma once
#include <array>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <iostream>
#include <map>
#include <string>
#include <vector>

namespace Eigen {
struct ThreadPoolDevice {};
template <typename T, std::size_t N> using array = std::array<T, N>;
// Only instantiated by the exact-float ("Null") kernels, which are never called.
struct half {
    float v;
    half() : v(0.f) {}
    half(int x) : v(float(x)) {}
    half(float x) : v(x) {}
    half &operator+=(const half &o) { v += o.v; return *this; }
    friend half operator*(const half &a, const half &b) { return half(a.v * b.v); }
};
}  // namespace Eigen

#define EIGEN_ALWAYS_INLINE inline

namespace tensorflow {
typedef std::uint8_t uint8;
typedef std::uint16_t uint16;
typedef std::uint32_t uint32;
typedef std::int64_t int64;

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
}  // namespace errors

// Attribute bag standing in for OpKernelConstruction.
class OpKernelConstruction {
public:
    std::map<std::string, int> int_attrs;
    std::map<std::string, std::string> string_attrs;
    Status status;
    Status GetAttr(const std::string &name, int *v) const {
        auto it = int_attrs.find(name);
        if (it == int_attrs.end()) return Status("missing attr " + name);
        *v = it->second;
        return Status::OK();
    }
    Status GetAttr(const std::string &name, std::string *v) const {
        auto it = string_attrs.find(name);
        if (it == string_attrs.end()) return Status("missing attr " + name);
        *v = it->second;
        return Status::OK();
    }
    void SetStatus(const Status &s) { if (status.ok()) status = s; }
};

// Scalar-only tensor: the reference reads inputs 2..5 as host float scalars.
class Tensor {
public:
    float value = 0.f;
    struct ScalarView {
        const float *p;
        float operator()() const { return *p; }
    };
    template <typename T> ScalarView scalar() const { return ScalarView{&value}; }
};

class OpKernelContext {
public:
    std::vector<Tensor> inputs;
    const Tensor &input(int i) const { return inputs[std::size_t(i)]; }
};

// Views used by the filter-sum functor (tf2/src/approx_nn_conv_kernels.cpp:300-306).
template <typename T> struct AxSumOverLeading3 {
    const T *data;
    long dims[4];
};
template <typename T> struct AxConstTensor4 {
    const T *data;
    long dims[4];
    AxSumOverLeading3<T> sum(const Eigen::array<int, 3> &) const {
        return AxSumOverLeading3<T>{data, {dims[0], dims[1], dims[2], dims[3]}};
    }
};
template <typename T> struct AxFlat {
    T *data;
    long size;
    void setZero() { for (long i = 0; i < size; ++i) data[i] = T(0); }
    struct OnDevice {
        AxFlat *self;
        void operator=(const AxSumOverLeading3<T> &e) {
            const long rows = e.dims[0] * e.dims[1] * e.dims[2], cols = e.dims[3];
            for (long j = 0; j < cols; ++j) {
                T s(0);
                for (long l = 0; l < rows; ++l) s += e.data[l * cols + j];
                self->data[j] = s;
            }
        }
    };
    OnDevice device(const Eigen::ThreadPoolDevice &) { return OnDevice{this}; }
};
template <typename T, int N = 1> struct TTypes {
    typedef AxFlat<T> Flat;
    typedef AxFlat<const T> ConstFlat;
    typedef AxConstTensor4<T> ConstTensor;
};
}  // namespace tensorflow

#define TF_PREDICT_TRUE(x) (x)
#define OP_REQUIRES_OK(CTX, ...)                         \
    do {                                                 \
        ::tensorflow::Status _s(__VA_ARGS__);            \
        if (!_s.ok()) { (CTX)->SetStatus(_s); return; }  \
    } while (0)
#define VLOG(n) if (true) {} else std::cerr
