// What the reference's Keras wrapper does before the op, on the device: the range of a tensor and the fake
// quantisation with that range (tf2/python/keras/layers/fake_approx_convolutional.py:233-242).  The range stays in
// device memory, where axc_conv2d_forward_device_ranges reads it: no host round trip between reduction and op.
#include <math_constants.h>

#include "axc_internal.h"

namespace axc {

namespace {

__global__ void range_reset_kernel(float *range2)
{
    range2[threadIdx.x] = threadIdx.x == 0 ? CUDART_INF_F : -CUDART_INF_F;
}

// min / max of floats with integer atomics on their bit patterns: non-negative floats order like signed integers,
// negative floats in reverse order of their unsigned patterns, so both extremes can be kept as plain floats in
// memory while blocks update them.
__device__ __forceinline__ void atomic_min_float(float *addr, float v)
{
    if (!(v < 0.0f) && !signbit(v)) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMax(reinterpret_cast<unsigned *>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_max_float(float *addr, float v)
{
    if (!(v < 0.0f) && !signbit(v)) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned *>(addr), __float_as_uint(v));
}

__global__ void __launch_bounds__(512) tensor_range_kernel(const float *__restrict__ x, size_t count, float *range2)
{
    float lo = CUDART_INF_F, hi = -CUDART_INF_F;
    const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, nthreads = size_t(gridDim.x) * blockDim.x;
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    const size_t quads = vec ? count / 4 : 0;
    for (size_t i = tid; i < quads; i += nthreads) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
        lo = fminf(fminf(lo, v.x), fminf(v.y, fminf(v.z, v.w)));      // fminf / fmaxf skip NaNs
        hi = fmaxf(fmaxf(hi, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
    }
    for (size_t i = quads * 4 + tid; i < count; i += nthreads) {
        const float v = __ldg(x + i);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    __shared__ float s_lo[16], s_hi[16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
    __syncthreads();
    if (warp == 0) {
        lo = lane < int(blockDim.x >> 5) ? s_lo[lane] : CUDART_INF_F;
        hi = lane < int(blockDim.x >> 5) ? s_hi[lane] : -CUDART_INF_F;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (lane == 0 && lo <= hi) {
            atomic_min_float(range2, lo);
            atomic_max_float(range2 + 1, hi);
        }
    }
}

// Forward of FakeQuantWithMinMaxVars (8 bits): nudged range as in tf2/src/approx_ops_types.h:29-49, then
// clamp, shift, scale, round half up, scale back - each a separately rounded fp32 operation.
__global__ void __launch_bounds__(256) fake_quant_kernel(const float *__restrict__ x, size_t count, const float *__restrict__ range2,
                                                         float *__restrict__ out)
{
    const float mn = range2[0], mx = range2[1];
    float scale = 0.0f, inv = 0.0f, nmin = 0.0f, nmax = 0.0f;
    const bool zero_range = mn == 0.0f && mx == 0.0f;
    if (!zero_range) {
        scale = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
        const float zp_from_min = __fsub_rn(0.0f, __fdiv_rn(mn, scale));
        float zp;
        if (zp_from_min < 0.0f) zp = 0.0f;
        else if (zp_from_min > 255.0f) zp = 255.0f;
        else zp = roundf(zp_from_min);
        nmin = __fmul_rn(__fsub_rn(0.0f, zp), scale);
        nmax = __fmul_rn(__fsub_rn(255.0f, zp), scale);
        inv = __fdiv_rn(1.0f, scale);
    }
    size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t nthreads = size_t(gridDim.x) * blockDim.x;
    for (; i < count; i += nthreads) {
        float y = 0.0f;
        if (!zero_range) {
            const float clamped = fminf(fmaxf(x[i], nmin), nmax);
            const float q = floorf(__fadd_rn(__fmul_rn(__fsub_rn(clamped, nmin), inv), 0.5f));
            y = __fadd_rn(__fmul_rn(q, scale), nmin);
        }
        out[i] = y;
    }
}

int with_device(int device, int *prev)
{
    AXC_CUDA(cudaGetDevice(prev));
    if (*prev != device) AXC_CUDA(cudaSetDevice(device));
    return AXC_OK;
}

}  // namespace

}  // namespace axc

extern "C" int axc_tensor_range(const float *x, size_t count, float *range2, int device, void *stream)
{
    using namespace axc;
    if (!range2 || (count > 0 && !x)) return AXC_INVALID_ARGUMENT;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    int prev = 0;
    rc = with_device(device, &prev);
    if (rc) return rc;
    cudaStream_t s = cudaStream_t(stream);
    range_reset_kernel<<<1, 2, 0, s>>>(range2);
    count_launch();
    if (count > 0) {
        const size_t want = (count / 4 + 511) / 512;
        const unsigned blocks = unsigned(want < size_t(di.sm_count) * 4 ? (want > 0 ? want : 1) : size_t(di.sm_count) * 4);
        tensor_range_kernel<<<blocks, 512, 0, s>>>(x, count, range2);
        count_launch();
    }
    const cudaError_t e = cudaGetLastError();
    if (prev != device) cudaSetDevice(prev);
    return e == cudaSuccess ? AXC_OK : cuda_failed(e);
}

extern "C" int axc_fake_quant(const float *x, size_t count, const float *range2, float *out, int device, void *stream)
{
    using namespace axc;
    if (!range2 || (count > 0 && (!x || !out))) return AXC_INVALID_ARGUMENT;
    if (count == 0) return AXC_OK;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    int prev = 0;
    rc = with_device(device, &prev);
    if (rc) return rc;
    const size_t want = (count + 255) / 256;
    const unsigned blocks = unsigned(want < size_t(di.sm_count) * 16 ? want : size_t(di.sm_count) * 16);
    fake_quant_kernel<<<blocks, 256, 0, cudaStream_t(stream)>>>(x, count, range2, out);
    count_launch();
    const cudaError_t e = cudaGetLastError();
    if (prev != device) cudaSetDevice(prev);
    return e == cudaSuccess ? AXC_OK : cuda_failed(e);
}

// ------------------------------------------------------------------------------------------------
// Max pooling, NHWC, SAME padding: one thread per output pixel and group of four channels (or one channel when the
// channel count or the pointers do not allow 16-byte accesses).
// ------------------------------------------------------------------------------------------------
namespace axc {
namespace {

template <int V>
__global__ void __launch_bounds__(256) max_pool_kernel(const float *__restrict__ in, float *__restrict__ out, int N, int H, int W,
                                                       int C, int OH, int OW, int k, int stride, int ph, int pw)
{
    const int cv = C / V;
    const long long total = (long long)N * OH * OW * cv;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int c = int(i % cv) * V;
        long long t = i / cv;
        const int ow = int(t % OW);
        t /= OW;
        const int oh = int(t % OH);
        const int n = int(t / OH);
        float m[V];
#pragma unroll
        for (int e = 0; e < V; ++e) m[e] = -INFINITY;
        for (int ky = 0; ky < k; ++ky) {
            const int iy = oh * stride - ph + ky;
            if (iy < 0 || iy >= H) continue;
            for (int kx = 0; kx < k; ++kx) {
                const int ix = ow * stride - pw + kx;
                if (ix < 0 || ix >= W) continue;
                const float *src = in + (((long long)n * H + iy) * W + ix) * C + c;
                if (V == 4) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(src));
                    m[0] = fmaxf(m[0], v.x); m[1 % V] = fmaxf(m[1 % V], v.y); m[2 % V] = fmaxf(m[2 % V], v.z); m[3 % V] = fmaxf(m[3 % V], v.w);
                } else {
                    m[0] = fmaxf(m[0], __ldg(src));
                }
            }
        }
        float *dst = out + (((long long)n * OH + oh) * OW + ow) * C + c;
        if (V == 4) *reinterpret_cast<float4 *>(dst) = make_float4(m[0], m[1 % V], m[2 % V], m[3 % V]);
        else dst[0] = m[0];
    }
}

}  // namespace
}  // namespace axc

extern "C" int axc_max_pool_same(const float *input, float *output, int n, int h, int w, int c, int k, int stride, int device,
                                 void *stream)
{
    using namespace axc;
    if (n < 0 || h <= 0 || w <= 0 || c <= 0 || k <= 0 || stride <= 0) return AXC_INVALID_ARGUMENT;
    const int oh = (h + stride - 1) / stride, ow = (w + stride - 1) / stride;
    if ((long long)n * oh * ow * c == 0) return AXC_OK;
    if (!input || !output) return AXC_INVALID_ARGUMENT;
    const int need_h = (oh - 1) * stride + k - h, need_w = (ow - 1) * stride + k - w;
    const int ph = (need_h > 0 ? need_h : 0) / 2, pw = (need_w > 0 ? need_w : 0) / 2;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    const bool vec = c % 4 == 0 && ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(output)) & 15u) == 0;
    const long long total = (long long)n * oh * ow * (vec ? c / 4 : c);
    const long long want = (total + 255) / 256;
    const unsigned blocks = unsigned(want < (long long)di.sm_count * 16 ? want : (long long)di.sm_count * 16);
    if (vec) max_pool_kernel<4><<<blocks, 256, 0, cudaStream_t(stream)>>>(input, output, n, h, w, c, oh, ow, k, stride, ph, pw);
    else max_pool_kernel<1><<<blocks, 256, 0, cudaStream_t(stream)>>>(input, output, n, h, w, c, oh, ow, k, stride, ph, pw);
    const cudaError_t e = cudaGetLastError();
    count_launch();
    if (prev != device) cudaSetDevice(prev);
    return e == cudaSuccess ? AXC_OK : cuda_failed(e);
}

