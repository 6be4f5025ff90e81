// Quantised entry point: uint8 operands in, int32 sums out - the contract of the reference's first-generation op
// `AxConv2D` (tf1/axqconv/axqconv.cc:66-94): every product of the integer convolution is a table lookup and the sum
// carries the zero-point corrections of the reference functor (tf1/axqconv/axqconv.cc:197-263)
//     total = sum_l ( LUT[a_l][b_l] - a_l * filter_offset - b_l * input_offset + input_offset * filter_offset ),
// where a tap outside the image has a_l = input_offset modulo 256: the functor stores the offset into its uint8
// operand type (:203-214), so an offset outside 0..255 (a range that does not contain 0) wraps there and only there.
//
// The table sums come from the same kernels as the fp32 op: the uint8 input is written out as fp32 values
// q - pad, pad = input_offset & 255, and the op is called with the range [-pad, 255 - pad], for which its quantiser
// has scale 1 and zero point `pad`: it maps q - pad back to q exactly, and 0.0 (a padded tap) to `pad`; the filter
// goes through as q with the range [0, 255].  The integer sums of the op (its accumulator tap) go straight to the
// caller's output; a second pass subtracts the zero-point terms.
#include "axc_internal.h"
#include "axc_sched.h"

namespace axc {

namespace {

__global__ void u8_to_grid_kernel(const uint8_t *__restrict__ q, long long n, int offset, float *__restrict__ out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = float(int(q[i]) - offset);
}

// bsum[j] = sum_l qfilter[l][j]
__global__ void qfilter_sum_kernel(const uint8_t *__restrict__ qf, int K, int Cout, int *__restrict__ bsum)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= Cout) return;
    int s = 0;
    for (int l = 0; l < K; ++l) s += int(qf[(size_t)l * Cout + j]);
    bsum[j] = s;
}

// psum[p] = sum_c qin[p][c] for every input pixel p (the zero-point terms need the sum of a patch's codes: nine of
// these for a 3x3 window instead of 9*C bytes)
__global__ void qpixel_sum_kernel(const uint8_t *__restrict__ q, long long pixels, int C, int vec_ok, int *__restrict__ psum)
{
    long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; p < pixels; p += stride) {
        const uint8_t *src = q + p * C;
        int s = 0;
        if (vec_ok) {
            const uint32_t *w = reinterpret_cast<const uint32_t *>(src);
            unsigned acc = 0;
            for (int c = 0; c < C / 4; ++c) acc = __dp4a(__ldg(w + c), 0x01010101u, acc);
            s = int(acc);
        } else {
            for (int c = 0; c < C; ++c) s += int(__ldg(src + c));
        }
        psum[p] = s;
    }
}

struct CorrParams {
    const int *psum;
    const int *bsum;
    int32_t *out;
    int N, H, W, C, KH, KW, Cout, sh, sw, dh, dw, ph, pw, OH, OW, K;
    long long M;
    int in_off, f_off, pad_code;
};

// One warp per output pixel: A = sum of the patch's quantised taps (pad_code where the tap is outside the image), one
// window position per lane, then out[p][j] += K*in_off*f_off - f_off*A - in_off*bsum[j] for all channels.
__global__ void __launch_bounds__(256) qconv_correct_kernel(const CorrParams P)
{
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int taps = P.KH * P.KW;
    for (long long p = warp0; p < P.M; p += nwarps) {
        const int ow = int(p % P.OW);
        const long long t = p / P.OW;
        const int oh = int(t % P.OH);
        const int n = int(t / P.OH);
        int a = 0;
        for (int tap = lane; tap < taps; tap += 32) {
            const int ky = tap / P.KW, kx = tap - ky * P.KW;
            const int iy = oh * P.sh - P.ph + ky * P.dh, ix = ow * P.sw - P.pw + kx * P.dw;
            const bool inside = iy >= 0 && iy < P.H && ix >= 0 && ix < P.W;
            a += inside ? __ldg(P.psum + ((long long)n * P.H + iy) * P.W + ix) : P.C * P.pad_code;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        const int base = P.K * P.in_off * P.f_off - P.f_off * a;
        int32_t *row = P.out + p * P.Cout;
        for (int j = lane; j < P.Cout; j += 32) row[j] += base - P.in_off * __ldg(P.bsum + j);
    }
}

size_t r256(size_t v) { return (v + 255) & ~size_t(255); }

struct QLayout {
    size_t dense_bytes, xin_off, xf_off, bsum_off, psum_off, total;
};

QLayout qconv_layout(const Geom &g)
{
    QLayout L;
    L.dense_bytes = r256(dense_workspace_total(g.K, g.Cout, g.M));
    L.xin_off = L.dense_bytes;
    L.xf_off = L.xin_off + r256(size_t(g.N) * g.H * g.W * g.C * 4);
    L.bsum_off = L.xf_off + r256(size_t(g.K) * g.Cout * 4);
    L.psum_off = L.bsum_off + r256(size_t(g.Cout) * 4);
    L.total = L.psum_off + r256(size_t(g.N) * g.H * g.W * 4);
    return L;
}

// The reference functor places the window with offsets of its own
// (tf1/axqconv/axqconv.cc:153-163): ((OW-1)*stride + KW - W [+ 1 for VALID]) / 2, truncated towards zero.  They equal
// TensorFlow's padding arithmetic, which this library applies, unless the stride exceeds the window by two or more;
// such shapes are refused rather than answered differently.
bool same_window_as_reference(const Geom &g, int padding)
{
    auto origin = [&](int out, int stride, int k, int in) { return ((out - 1) * stride + k - in + (padding == AXC_PADDING_VALID ? 1 : 0)) / 2; };
    return origin(g.OW, g.sw, g.KW, g.W) == g.pw && origin(g.OH, g.sh, g.KH, g.H) == g.ph;
}

}  // namespace

}  // namespace axc

extern "C" int axc_qconv2d_workspace_bytes(const axc_conv_desc *desc, size_t *bytes)
{
    if (!bytes) return AXC_INVALID_ARGUMENT;
    axc::Geom g;
    int rc = axc::resolve_geometry(desc, false, &g);
    if (rc) return rc;
    *bytes = axc::qconv_layout(g).total;
    return AXC_OK;
}

extern "C" int axc_qconv2d_forward(axc_table *table, const axc_conv_desc *desc, const uint8_t *qinput, const uint8_t *qfilter,
                                   int32_t input_offset, int32_t filter_offset, int32_t *output, void *workspace,
                                   size_t workspace_bytes, int device, void *stream)
{
    using namespace axc;
    if (!table || !desc) return AXC_INVALID_ARGUMENT;
    Geom g;
    int rc = resolve_geometry(desc, false, &g);
    if (rc) return rc;
    if (g.M * g.Cout == 0) return AXC_OK;
    if (!qinput || !qfilter || !output) return AXC_INVALID_ARGUMENT;
    {
        // the reference's int32 total must not overflow: bound every term of the sum
        const long long ai = input_offset < 0 ? -(long long)input_offset : input_offset, af = filter_offset < 0 ? -(long long)filter_offset : filter_offset;
        const long long mi = ai > 255 ? ai : 255, mf = af > 255 ? af : 255;
        if (mi > 0x7FFFFFFFll / mf || (long long)g.K > 0x7FFFFFFFll / (mi * mf)) return AXC_INVALID_ARGUMENT;
    }
    const int pad_code = input_offset & 255;
    // AxQuantizedConv2DOp accepts equal strides and no dilation only (tf1/axqconv/axqconv.cc:305-326)
    if (g.sh != g.sw || g.dh != 1 || g.dw != 1) return AXC_INVALID_ARGUMENT;
    if (!same_window_as_reference(g, desc->padding)) return AXC_UNIMPLEMENTED;
    if (!table_sum_fits_int32(table, g.K)) return AXC_INVALID_ARGUMENT;
    const QLayout L = qconv_layout(g);
    if (!workspace || workspace_bytes < L.total) return AXC_INTERNAL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return AXC_INVALID_ARGUMENT;
    int status = AXC_OK;
    const uint16_t *lut = table_device_ptr(table, device, &status);
    if (status) return status;

    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    cudaStream_t s = cudaStream_t(stream);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    float *xin = reinterpret_cast<float *>(ws + L.xin_off);
    float *xf = reinterpret_cast<float *>(ws + L.xf_off);
    int *bsum = reinterpret_cast<int *>(ws + L.bsum_off);
    const long long n_in = (long long)g.N * g.H * g.W * g.C, n_f = (long long)g.K * g.Cout;
    auto blocks = [](long long n) { return unsigned(n / 256 + 1 < 8192 ? n / 256 + 1 : 8192); };
    u8_to_grid_kernel<<<blocks(n_in), 256, 0, s>>>(qinput, n_in, pad_code, xin);
    u8_to_grid_kernel<<<blocks(n_f), 256, 0, s>>>(qfilter, n_f, 0, xf);
    cudaError_t e = cudaGetLastError();
    count_launch(2);
    if (e == cudaSuccess) {
        // scale 1, zero point = pad_code: the op's quantiser returns the caller's bytes, and pad_code for a padded tap
        const Quant q = make_quant(float(-pad_code), float(255 - pad_code), 0.0f, 255.0f);
        axc_debug_out taps = {nullptr, nullptr, output};
        Geom ge = g;
        ge.accum = AXC_ACCUM_EXACT_I32;
        ge.plan = g.plan;
        rc = launch_dense(lut, table_uid(table), ge, q, nullptr, xin, xf, nullptr, ws, &taps, device, s, false);
    }
    if (e == cudaSuccess && rc == AXC_OK && (input_offset != 0 || filter_offset != 0)) {
        qfilter_sum_kernel<<<unsigned((g.Cout + 127) / 128), 128, 0, s>>>(qfilter, g.K, g.Cout, bsum);
        int *psum = reinterpret_cast<int *>(ws + L.psum_off);
        const long long pixels = (long long)g.N * g.H * g.W;
        const int vec_ok = (g.C % 4 == 0 && (reinterpret_cast<uintptr_t>(qinput) & 3u) == 0) ? 1 : 0;
        qpixel_sum_kernel<<<blocks(pixels), 256, 0, s>>>(qinput, pixels, g.C, vec_ok, psum);
        CorrParams P;
        P.psum = psum; P.bsum = bsum; P.out = output;
        P.N = g.N; P.H = g.H; P.W = g.W; P.C = g.C; P.KH = g.KH; P.KW = g.KW; P.Cout = g.Cout;
        P.sh = g.sh; P.sw = g.sw; P.dh = g.dh; P.dw = g.dw; P.ph = g.ph; P.pw = g.pw; P.OH = g.OH; P.OW = g.OW; P.K = g.K;
        P.M = g.M; P.in_off = input_offset; P.f_off = filter_offset; P.pad_code = pad_code;
        const long long warps = g.M;
        qconv_correct_kernel<<<unsigned(warps / 8 + 1 < 16384 ? warps / 8 + 1 : 16384), 256, 0, s>>>(P);
        e = cudaGetLastError();
        count_launch(3);
    }
    if (prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_failed(e);
    return rc;
}

// FloatToQuantizedUnclamped<quint8>(0.0f, min, max): the code that stands for the real value 0
// (tf1/axqconv/quantization_utils.h:49-64, called at tf1/axqconv/axqconv.cc:365-368).
extern "C" int axc_quantized_zero_point(float range_min, float range_max, int32_t *offset)
{
    if (!offset) return AXC_INVALID_ARGUMENT;
    if (range_min == range_max) {
        *offset = 0;
        return AXC_OK;
    }
    const double steps = 256.0;
    const double range_adjust = steps / (steps - 1.0);
    volatile float span = range_max - range_min;          // a float subtraction, as in the reference
    const double range = double(span) * range_adjust;
    const double range_scale = steps / range;
    *offset = int32_t((long long)(__builtin_round(0.0 * range_scale) - __builtin_round(double(range_min) * range_scale)));
    return AXC_OK;
}

// QuantizationRangeForMultiplication<quint8, quint8, qint32> (tf1/axqconv/quantization_utils.h:116-140, called at
// tf1/axqconv/axqconv.cc:429-441): the real values that the int32 codes lowest and highest stand for.
extern "C" int axc_quantized_output_range(float min_a, float max_a, float min_b, float max_b, float out2[2])
{
    if (!out2) return AXC_INVALID_ARGUMENT;
    volatile float a_level = (max_a - min_a) / 255.0f;
    volatile float b_level = (max_b - min_b) / 255.0f;
    volatile float c_level = a_level * b_level;
    out2[0] = c_level * float(-2147483647ll - 1);
    out2[1] = c_level * float(2147483647ll);
    return AXC_OK;
}
