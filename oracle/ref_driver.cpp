// TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
//
// C entry points around the reference's own CPU table kernels.  This file is
// compiled together with the reference translation unit
// tf2/src/approx_nn_conv_kernels.cpp (taken from the reference checkout where it
// lies; never copied) against the stand-in headers in oracle/tf_stub/.
// The arithmetic that runs - Nudge/Update (tf2/src/approx_ops_types.h:29-49,
// 135-197), table loading (:99-122, 205-216), the patch builder, the table GEMM,
// the fused GEMM and the filter sums (tf2/src/approx_nn_conv_kernels.cpp:167-306)
// - is the reference's code.  Only the launcher's dispatch and chunk loop
// (tf2/src/approx_nn_conv_ops.cpp:70-206) and TF's window arithmetic are
// restated here, because that file needs the full TensorFlow runtime.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "approx_nn_conv_kernels.h"

using CPUDevice = Eigen::ThreadPoolDevice;
using RefOp = TableApproxOpType_t<CPUDevice, float, tensorflow::uint8>;

namespace {
struct Handle {
    tensorflow::OpKernelConstruction ctor;
    RefOp *op = nullptr;
};

int window(int in, int k, int dil, int stride, int padding, int *out, int *pad_before)
{
    const int eff = (k - 1) * dil + 1;
    if (padding == 1) {
        *out = (in - eff + stride) / stride;
        *pad_before = 0;
    } else {
        *out = (in + stride - 1) / stride;
        *pad_before = std::max((*out - 1) * stride + eff - in, 0) / 2;
    }
    return *out < 0 ? 3 : 0;
}
}  // namespace

extern "C" {

// Returns NULL when the reference constructor reports an error (unreadable table).
void *axr_create(const char *mul_map_file, int num_bits)
{
    Handle *h = new Handle;
    h->ctor.int_attrs["num_bits"] = num_bits;
    h->ctor.string_attrs["mul_map_file"] = mul_map_file ? mul_map_file : "";
    h->op = new RefOp(&h->ctor);
    if (!h->ctor.status.ok()) {
        delete h->op;
        delete h;
        return nullptr;
    }
    return h;
}

void axr_destroy(void *hv)
{
    Handle *h = static_cast<Handle *>(hv);
    if (!h) return;
    delete h->op;
    delete h;
}

void axr_update(void *hv, float in_min, float in_max, float f_min, float f_max)
{
    Handle *h = static_cast<Handle *>(hv);
    tensorflow::OpKernelContext ctx;
    ctx.inputs.resize(6);
    ctx.inputs[2].value = in_min;
    ctx.inputs[3].value = in_max;
    ctx.inputs[4].value = f_min;
    ctx.inputs[5].value = f_max;
    h->op->Update(&ctx);
}

// out[10] = input{scale,inv,offset}, filter{scale,inv,offset}, s1s2, m1, m2, m1m2
void axr_get_quant(void *hv, float *out)
{
    const auto &q = static_cast<Handle *>(hv)->op->quantProps;
    out[0] = q.input.scale; out[1] = q.input.invScale; out[2] = q.input.offset;
    out[3] = q.filter.scale; out[4] = q.filter.invScale; out[5] = q.filter.offset;
    out[6] = q.s1xS2; out[7] = q.m1; out[8] = q.m2; out[9] = q.m1xM2;
}

void axr_get_table(void *hv, uint16_t *out)
{
    const auto &t = static_cast<Handle *>(hv)->op->lookupTable;
    std::memcpy(out, t.data(), t.size() * sizeof(uint16_t));
}

void axr_im2col(void *hv, const float *in, int c, int w, int h, int ow, int oh, int kw, int kh,
                int pw, int ph, int sw, int sh, int dw, int dh, int po, int pc,
                uint8_t *out, float *out_coeffs)
{
    CPUDevice d;
    ApproxConvIm2ColKernel<CPUDevice, float, tensorflow::uint8, TableApproxOpType_t>()(
        d, *static_cast<Handle *>(hv)->op, in, c, w, h, ow, oh, kw, kh, pw, ph, sw, sh, dw, dh, po, pc,
        out, out_coeffs);
}

void axr_gemm(void *hv, int m, int n, int k, const uint8_t *a, const float *b,
              const float *a_coeffs, const float *b_coeffs, float *c)
{
    CPUDevice d;
    ApproxConvGEMMKernel<CPUDevice, float, tensorflow::uint8, TableApproxOpType_t>()(
        d, *static_cast<Handle *>(hv)->op, m, n, k, 0.f, a, k, b, n, a_coeffs, b_coeffs, 0.f, c, n);
}

void axr_gemm_combined(void *hv, int m, int n, int k, const float *a, const float *b, float *c)
{
    CPUDevice d;
    ApproxConvGEMMKernelCombined<CPUDevice, float, tensorflow::uint8, TableApproxOpType_t>()(
        d, *static_cast<Handle *>(hv)->op, m, n, k, 0.f, a, k, b, n, 0.f, c, n);
}

void axr_filter_sums(void *hv, const float *filter, int kh, int kw, int c, int n, float *out)
{
    CPUDevice d;
    ConstTensor4<float> f{filter, {kh, kw, c, n}};
    Flat<float> o{out, n};
    ApproxFilterCorrCoeff<CPUDevice, float, tensorflow::uint8, TableApproxOpType_t>()(
        d, *static_cast<Handle *>(hv)->op, f, o);
}

// Whole forward pass: dispatch and 16 MiB chunking as in
// tf2/src/approx_nn_conv_ops.cpp:70-206, kernels from the reference.
// padding: 0 SAME, 1 VALID.  Returns 0, or 3 (InvalidArgument).
int axr_conv2d(void *hv, int n, int h, int w, int c, int kh, int kw, int cout,
               int stride_h, int stride_w, int dil_h, int dil_w, int padding,
               const float *input, const float *filter,
               float in_min, float in_max, float f_min, float f_max, float *output)
{
    int oh, ow, ph, pw;
    if (window(h, kh, dil_h, stride_h, padding, &oh, &ph)) return 3;
    if (window(w, kw, dil_w, stride_w, padding, &ow, &pw)) return 3;
    const int64_t total = int64_t(n) * oh * ow;
    if (total == 0 || cout == 0) return 0;
    axr_update(hv, in_min, in_max, f_min, f_max);

    if (kh == 1 && kw == 1 && stride_h == 1 && stride_w == 1) {
        axr_gemm_combined(hv, int(int64_t(n) * h * w), cout, c, input, filter, output);
        return 0;
    }
    if (kh == h && kw == w && dil_h == 1 && dil_w == 1 && padding == 1) {
        axr_gemm_combined(hv, n, cout, int(int64_t(h) * w * c), input, filter, output);
        return 0;
    }
    const int64_t max_chunk = (16 * 1024 * 1024) / int64_t(sizeof(float));
    const int64_t patch_len = int64_t(kh) * kw * c;
    if (patch_len > max_chunk) return 3;
    const int64_t per_chunk = max_chunk / patch_len;
    std::vector<uint8_t> a(static_cast<size_t>(max_chunk));
    std::vector<float> a_sum(static_cast<size_t>(per_chunk)), b_sum(static_cast<size_t>(cout));
    axr_filter_sums(hv, filter, kh, kw, c, cout, b_sum.data());
    float *out_p = output;
    for (int64_t i = 0; i < total; i += per_chunk) {
        const int64_t batch = i / (int64_t(oh) * ow);
        const int patch_off = int(i % (int64_t(oh) * ow));
        const int pc = int(std::min(per_chunk, total - i));
        const float *in_b = input + batch * h * w * c;
        axr_im2col(hv, in_b, c, w, h, ow, oh, kw, kh, pw, ph, stride_w, stride_h, dil_w, dil_h,
                   patch_off, pc, a.data(), a_sum.data());
        axr_gemm(hv, pc, cout, int(patch_len), a.data(), filter, a_sum.data(), b_sum.data(), out_p);
        out_p += per_chunk * cout;
    }
    return 0;
}

}  // extern "C"
