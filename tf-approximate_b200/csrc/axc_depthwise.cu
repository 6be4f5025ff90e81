// Depthwise table-driven convolution for sm_100a.
//
// The reference has no grouped path (it rejects such shapes,
// tf2/src/approx_nn_conv_ops.cpp:229-232); this kernel applies the reference's per-MAC rule
// (quantiser, table index, dequantisation: tf2/src/approx_nn_conv_kernels.cpp:167-211) to
// TensorFlow's depthwise layout: filter [KH,KW,C,mult], output channel c*mult + m, K = KH*KW.
//
// Lane = output channel (consecutive channels are contiguous in NHWC, so every global
// access of a warp is one 128-byte line), one warp walks a run of output pixels of one
// image row and keeps the 3x3 input window in registers, so an input element is read once
// per output row it touches; the new window columns of four outputs are requested together.  The table lives in shared memory in the two-plane layout of
// the dense kernel (plane p at 65536*(1+p), byte a*256 + 2*(b&127)).
#include <mutex>

#include "axc_internal.h"

namespace axc {

namespace {

constexpr int kDwThreads = 1024;
constexpr int kDwWarps = kDwThreads / 32;
constexpr unsigned kLutBase = 65536u;
constexpr unsigned kSmemEnd = 196608u;

struct DwParams {
    const uint16_t *lut;
    const float *input;
    float *output;
    const uint32_t *prog;  // [KH*KW][OC] program words {2*(b&127), 0, 1+(b>>7), 0}
    const float *bsum;     // [OC]
    int32_t *acc_out;
    int *status;
    int N, H, W, C, KH, KW, mult, OC;
    int sh, sw, dh, dw, ph, pw, OH, OW;
    int run;               // output pixels per warp item
    int runs_per_row, groups;
    long long items;       // N*OH*runs_per_row*groups
    float in_off, in_inv, s1s2, m1, m2, km1m2;
};

__device__ __forceinline__ unsigned dw_quantize_u8(float x, float off, float inv)
{
    const float v = __fadd_rn(__fmul_rn(__fsub_rn(x, off), inv), 0.5f);
    const unsigned u = __float2uint_rz(v);
    return u > 255u ? 255u : u;
}

__device__ __forceinline__ unsigned dw_lds_u16(unsigned addr)
{
    unsigned v;
    asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Quantise the depthwise filter [KHW][OC] into program words, the plain uint8 copy
// (optional) and the per-channel fp32 filter sums (tap order).
__global__ void dw_filter_prep_kernel(const float *__restrict__ filter, int KHW, int OC, float f_off, float f_inv,
                                      uint32_t *__restrict__ prog, float *__restrict__ bsum,
                                      uint8_t *__restrict__ qfilter, int *status)
{
    const int oc = blockIdx.x * blockDim.x + threadIdx.x;
    if (oc == 0) *status = 0;
    if (oc >= OC) return;
    float s = 0.0f;
    for (int t = 0; t < KHW; ++t) {
        const float f = filter[(size_t)t * OC + oc];
        s = __fadd_rn(s, f);
        const unsigned b = dw_quantize_u8(f, f_off, f_inv);
        prog[(size_t)t * OC + oc] = ((b & 127u) << 1) | ((1u + (b >> 7)) << 16);
        if (qfilter) qfilter[(size_t)t * OC + oc] = uint8_t(b);
    }
    bsum[oc] = s;
}

__global__ void dw_quantize_tensor_kernel(const float *__restrict__ x, long long n, float off, float inv,
                                          uint8_t *__restrict__ q)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) q[i] = uint8_t(dw_quantize_u8(x[i], off, inv));
}

__device__ __forceinline__ void dw_fill_table(const uint16_t *lut, int tid, int nthreads)
{
    const uint4 *src = reinterpret_cast<const uint4 *>(lut);
    for (int i = tid; i < 8192; i += nthreads) {
        const int a = i >> 5, part = i & 31;
        const uint4 v = __ldg(src + i);
        const unsigned dst = kLutBase + (part >= 16 ? 65536u : 0u) + unsigned(a) * 256u + unsigned(part & 15) * 16u;
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
}

__device__ __forceinline__ float dw_epilogue(int acc, float a_sum, float t2, const DwParams &P)
{
    const float t0 = __fmul_rn(float(acc), P.s1s2);
    const float t1 = __fmul_rn(P.m2, a_sum);
    return __fsub_rn(__fadd_rn(__fadd_rn(t0, t1), t2), P.km1m2);
}

// Any KH x KW, stride and dilation: every tap is fetched for every output.
__global__ void __launch_bounds__(kDwThreads, 1) depthwise_generic_kernel(const DwParams P)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const unsigned dyn0 = (unsigned)__cvta_generic_to_shared(smem_raw);
    unsigned dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (dyn0 > kLutBase || dyn0 + dyn_size < kSmemEnd) {
        if (threadIdx.x == 0) atomicExch(P.status, 1);
        return;
    }
    dw_fill_table(P.lut, threadIdx.x, kDwThreads);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int khw = P.KH * P.KW;
    for (long long item = (long long)blockIdx.x * kDwWarps + warp; item < P.items; item += (long long)gridDim.x * kDwWarps) {
        const int grp = int(item % P.groups);
        long long t = item / P.groups;
        const int r = int(t % P.runs_per_row);
        t /= P.runs_per_row;
        const int oh = int(t % P.OH);
        const int n = int(t / P.OH);
        const int oc = grp * 32 + lane;
        if (oc >= P.OC) continue;
        const int c = oc / P.mult;
        const float t2 = __fmul_rn(P.m1, __ldg(P.bsum + oc));
        const int ow_end = min(P.OW, (r + 1) * P.run);
        for (int ow = r * P.run; ow < ow_end; ++ow) {
            int acc = 0;
            float a_sum = 0.0f;
            for (int tap = 0; tap < khw; ++tap) {
                const int ky = tap / P.KW, kx = tap - ky * P.KW;
                const int iy = oh * P.sh - P.ph + ky * P.dh, ix = ow * P.sw - P.pw + kx * P.dw;
                float v = 0.0f;
                if (iy >= 0 && iy < P.H && ix >= 0 && ix < P.W)
                    v = __ldg(P.input + (((long long)n * P.H + iy) * P.W + ix) * P.C + c);
                a_sum = __fadd_rn(a_sum, v);
                const unsigned qa = dw_quantize_u8(v, P.in_off, P.in_inv);
                const unsigned w = __ldg(P.prog + (size_t)tap * P.OC + oc);
                acc += int(dw_lds_u16(__byte_perm(w, qa, 0x3240)));
            }
            const long long o = (((long long)n * P.OH + oh) * P.OW + ow) * P.OC + oc;
            P.output[o] = dw_epilogue(acc, a_sum, t2, P);
            if (P.acc_out) P.acc_out[o] = acc;
        }
    }
}

// 3x3, dilation 1, stride S in {1, 2}: sliding window of raw and quantised taps in registers.
template <int S>
__global__ void __launch_bounds__(kDwThreads, 1) depthwise_3x3_kernel(const DwParams P)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const unsigned dyn0 = (unsigned)__cvta_generic_to_shared(smem_raw);
    unsigned dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (dyn0 > kLutBase || dyn0 + dyn_size < kSmemEnd) {
        if (threadIdx.x == 0) atomicExch(P.status, 1);
        return;
    }
    dw_fill_table(P.lut, threadIdx.x, kDwThreads);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long item = (long long)blockIdx.x * kDwWarps + warp; item < P.items; item += (long long)gridDim.x * kDwWarps) {
        const int grp = int(item % P.groups);
        long long t = item / P.groups;
        const int r = int(t % P.runs_per_row);
        t /= P.runs_per_row;
        const int oh = int(t % P.OH);
        const int n = int(t / P.OH);
        const int oc = grp * 32 + lane;
        if (oc >= P.OC) continue;
        const int c = oc / P.mult;
        const float t2 = __fmul_rn(P.m1, __ldg(P.bsum + oc));
        unsigned w[9];
#pragma unroll
        for (int tap = 0; tap < 9; ++tap) w[tap] = __ldg(P.prog + (size_t)tap * P.OC + oc);

        const int iy0 = oh * P.sh - P.ph;
        const float *rowp[3];
        bool rowok[3];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const int iy = iy0 + ky;
            rowok[ky] = iy >= 0 && iy < P.H;
            rowp[ky] = P.input + (((long long)n * P.H + (rowok[ky] ? iy : 0)) * P.W) * P.C + c;
        }
        auto fetch = [&](int ky, int ix) -> float {
            return (rowok[ky] && ix >= 0 && ix < P.W) ? __ldg(rowp[ky] + (long long)ix * P.C) : 0.0f;
        };

        const int ow0 = r * P.run;
        const int ow_end = min(P.OW, ow0 + P.run);
        float xf[3][3];
        unsigned xq[3][3];
        // columns 0 .. 2-S of the first window come from the "previous" position
        const int ix_first = ow0 * S - P.pw;
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
            for (int kx = S; kx < 3; ++kx) {
                xf[ky][kx] = fetch(ky, ix_first + kx - S);
                xq[ky][kx] = dw_quantize_u8(xf[ky][kx], P.in_off, P.in_inv);
            }
        // Outputs are produced in batches: the new input columns of a whole batch are requested first, so that
        // kBatch * S * 3 loads per lane are in flight while the previous values are consumed.
        constexpr int kBatch = 4;
        for (int owb = ow0; owb < ow_end; owb += kBatch) {
            float nf[kBatch][3][S];
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
#pragma unroll
                for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                    for (int k2 = 0; k2 < S; ++k2)
                        nf[u][ky][k2] = (owb + u < ow_end) ? fetch(ky, (owb + u) * S - P.pw + (3 - S) + k2) : 0.0f;
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int ow = owb + u;
                if (ow < ow_end) {
                    // shift the window left by S columns, append the S new columns
#pragma unroll
                    for (int ky = 0; ky < 3; ++ky) {
#pragma unroll
                        for (int kx = 0; kx < 3 - S; ++kx) {
                            xf[ky][kx] = xf[ky][kx + S];
                            xq[ky][kx] = xq[ky][kx + S];
                        }
#pragma unroll
                        for (int k2 = 0; k2 < S; ++k2) {
                            xf[ky][3 - S + k2] = nf[u][ky][k2];
                            xq[ky][3 - S + k2] = dw_quantize_u8(nf[u][ky][k2], P.in_off, P.in_inv);
                        }
                    }
                    int acc = 0;
                    float a_sum = 0.0f;
#pragma unroll
                    for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                        for (int kx = 0; kx < 3; ++kx) {
                            a_sum = __fadd_rn(a_sum, xf[ky][kx]);
                            acc += int(dw_lds_u16(__byte_perm(w[ky * 3 + kx], xq[ky][kx], 0x3240)));
                        }
                    const long long o = (((long long)n * P.OH + oh) * P.OW + ow) * P.OC + oc;
                    P.output[o] = dw_epilogue(acc, a_sum, t2, P);
                    if (P.acc_out) P.acc_out[o] = acc;
                }
            }
        }
    }
}

template <typename Kern>
int launch_dw(Kern kern, const DwParams &P, const DeviceInfo &di, cudaStream_t stream)
{
    AXC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
    const long long ctas_needed = (P.items + kDwWarps - 1) / kDwWarps;
    const long long grid = ctas_needed < di.sm_count ? ctas_needed : di.sm_count;
    kern<<<unsigned(grid), kDwThreads, size_t(di.max_smem_optin), stream>>>(P);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    return AXC_OK;
}

}  // namespace

int launch_depthwise(const uint16_t *lut_dev, const Geom &g, const Quant &q, const float *input,
                     const float *filter, float *output, void *workspace, const axc_debug_out *dbg,
                     int device, cudaStream_t stream)
{
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    if (di.max_smem_optin < int(kSmemEnd)) return AXC_INTERNAL;
    const int OC = g.C * g.Cout;
    const Workspace ws = depthwise_workspace(g.K, g.C, g.Cout);
    unsigned char *wsb = static_cast<unsigned char *>(workspace);
    uint32_t *prog = reinterpret_cast<uint32_t *>(wsb);
    float *bsum = reinterpret_cast<float *>(wsb + ws.sums_off);
    int *status = reinterpret_cast<int *>(wsb + ws.status_off);

    dw_filter_prep_kernel<<<unsigned((OC + 127) / 128), 128, 0, stream>>>(filter, g.K, OC, q.f_off, q.f_inv, prog, bsum,
                                                                         dbg ? dbg->qfilter : nullptr, status);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    if (dbg && dbg->qinput) {
        const long long n = (long long)g.N * g.H * g.W * g.C;
        if (n > 0) {
            const unsigned blocks = unsigned(n / 256 + 1 < 4096 ? n / 256 + 1 : 4096);
            dw_quantize_tensor_kernel<<<blocks, 256, 0, stream>>>(input, n, q.in_off, q.in_inv, dbg->qinput);
            AXC_CUDA(cudaGetLastError());
            count_launch();
        }
    }

    DwParams P;
    P.lut = lut_dev; P.input = input; P.output = output; P.prog = prog; P.bsum = bsum;
    P.acc_out = dbg ? dbg->acc : nullptr;
    P.status = status;
    P.N = g.N; P.H = g.H; P.W = g.W; P.C = g.C; P.KH = g.KH; P.KW = g.KW; P.mult = g.Cout; P.OC = OC;
    P.sh = g.sh; P.sw = g.sw; P.dh = g.dh; P.dw = g.dw; P.ph = g.ph; P.pw = g.pw; P.OH = g.OH; P.OW = g.OW;
    P.run = g.OW < 16 ? g.OW : 16;   // a multiple of the 3x3 kernels' batch of four outputs
    P.runs_per_row = (g.OW + P.run - 1) / P.run;
    P.groups = (OC + 31) / 32;
    P.items = (long long)g.N * g.OH * P.runs_per_row * P.groups;
    P.in_off = q.in_off; P.in_inv = q.in_inv; P.s1s2 = q.s1s2; P.m1 = q.m1; P.m2 = q.m2;
    {
        volatile float kf = float(g.K);
        volatile float t3 = kf * q.m1m2;
        P.km1m2 = t3;
    }
    const bool k3 = g.KH == 3 && g.KW == 3 && g.dh == 1 && g.dw == 1 && g.sh == g.sw;
    if (k3 && g.sw == 1) return launch_dw(depthwise_3x3_kernel<1>, P, di, stream);
    if (k3 && g.sw == 2) return launch_dw(depthwise_3x3_kernel<2>, P, di, stream);
    return launch_dw(depthwise_generic_kernel, P, di, stream);
}

// ---------------------------------------------------------------------------------------------------
// Entry point that allocates nothing: the scratch of the depthwise path (filter program words, filter
// sums, status word) lives in a file-scope device array instead of a caller-provided workspace.
// ---------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = size_t(1) << 20;   // 1 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_dw_static_scratch[kStaticScratchBytes];

// Device address of g_dw_static_scratch on `device` (which must be current).  In host code the array's name
// is only a handle for the runtime, not an address a kernel could use, so the address is asked for once per
// device and remembered.
int static_scratch_address(int device, void **out)
{
    static std::mutex mu;
    static void *addr[64] = {};
    if (device < 0 || device >= 64) return AXC_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[device]) {
        void *p = nullptr;
        AXC_CUDA(cudaGetSymbolAddress(&p, g_dw_static_scratch));
        addr[device] = p;
    }
    *out = addr[device];
    return AXC_OK;
}

}  // namespace

}  // namespace axc

extern "C" int axc_depthwise_conv2d_forward_noalloc(axc_table *table, const axc_conv_desc *desc, const float *input,
                                                    const float *filter, float in_min, float in_max, float f_min,
                                                    float f_max, float *output, int device, void *stream)
{
    using namespace axc;
    if (!table || !desc) return AXC_INVALID_ARGUMENT;
    Geom g;
    int rc = resolve_geometry(desc, true, &g);
    if (rc) return rc;
    if (g.M * (long long)g.C * g.Cout == 0) return AXC_OK;
    if (!input || !filter || !output) return AXC_INVALID_ARGUMENT;
    // the scratch this shape needs must fit the fixed array
    if (depthwise_workspace(g.K, g.C, g.Cout).total > kStaticScratchBytes) return AXC_INVALID_ARGUMENT;
    const uint16_t *lut = table_device_ptr_if_resident(table, device);
    if (!lut) return AXC_INTERNAL;   // axc_table_ensure_device(table, device) has to run first: it allocates
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    void *scratch = nullptr;
    rc = static_scratch_address(device, &scratch);
    if (rc == AXC_OK) {
        const Quant q = make_quant(in_min, in_max, f_min, f_max);
        rc = launch_depthwise(lut, g, q, input, filter, output, scratch, nullptr, device, cudaStream_t(stream));
    }
    if (prev != device) cudaSetDevice(prev);
    return rc;
}
