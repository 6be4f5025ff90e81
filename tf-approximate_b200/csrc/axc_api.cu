// Host side of libaxconv: truth tables, geometry, quantisation parameters and the C ABI.
// No TensorFlow, no torch: plain CUDA runtime.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "axc_internal.h"
#include "axc_sched.h"

struct axc_table {
    unsigned uid;
    uint32_t max_entry;          // largest entry
    int common_tz;               // trailing zero bits shared by all entries (16 for an all-zero table)
    std::vector<uint16_t> host;  // 65536 entries, index (a << 8) | b
    std::mutex mu;
    std::vector<uint16_t *> dev;  // per-device replica, lazily created
};

namespace axc {

static thread_local int g_last_cuda_error = 0;
static std::atomic<uint64_t> g_launches{0};
static std::atomic<unsigned> g_table_uid{1};

unsigned table_uid(const axc_table *t) { return t->uid; }
void stamp(axc_table *t)
{
    t->uid = g_table_uid.fetch_add(1);
    uint32_t mx = 0, ored = 0;
    for (uint16_t v : t->host) {
        mx = v > mx ? v : mx;
        ored |= v;
    }
    t->max_entry = mx;
    int tz = 0;
    while (tz < 16 && ((ored >> tz) & 1u) == 0u) ++tz;
    t->common_tz = tz;
}

bool table_sum_exact_in_fp32(const axc_table *t, long long K)
{
    if (t->max_entry == 0) return true;
    // K <= 2^22 here (resolve_geometry) and max_entry < 2^16: the product fits 64 bits with room
    return K * (long long)t->max_entry <= (1ll << (24 + t->common_tz));
}

bool table_sum_fits_int32(const axc_table *t, long long K)
{
    return K * (long long)t->max_entry <= 0x7FFFFFFFll;
}

int cuda_failed(cudaError_t e)
{
    g_last_cuda_error = int(e);
    return AXC_CUDA_ERROR;
}

void count_launch(int n) { g_launches.fetch_add(uint64_t(n), std::memory_order_relaxed); }

// Range nudging of TensorFlow's fake-quant as the reference restates it
// (tf2/src/approx_ops_types.h:29-49) and the zero-range rule of
// UpdateVarQuantProps (:135-152).  Every operation is a separately rounded fp32
// operation; the volatile stores keep the host compiler from fusing them.
void var_quant_props(float min_v, float max_v, float *scale, float *inv, float *offset)
{
    volatile float s = 0.0f, i = 0.0f, nudged_min = 0.0f;
    if (min_v != 0.0f || max_v != 0.0f) {
        const float qmin = 0.0f, qmax = 255.0f;
        s = (max_v - min_v) / (qmax - qmin);
        volatile float ratio = min_v / s;
        volatile float zp_from_min = qmin - ratio;
        uint16_t zp;
        if (zp_from_min < qmin)
            zp = 0;
        else if (zp_from_min > qmax)
            zp = 255;
        else
            zp = uint16_t(std::round(zp_from_min));
        // a true subtraction: 0 - 0 must give +0.0 as in the reference, not the -0.0 of a negation
        volatile float zp_f = float(zp), zero = qmin;
        volatile float neg_zp = zero - zp_f;
        nudged_min = neg_zp * s;
        i = 1.0f / s;
    }
    *scale = s;
    *inv = i;
    *offset = nudged_min;
}

Quant make_quant(float in_min, float in_max, float f_min, float f_max)
{
    Quant q;
    var_quant_props(in_min, in_max, &q.in_scale, &q.in_inv, &q.in_off);
    var_quant_props(f_min, f_max, &q.f_scale, &q.f_inv, &q.f_off);
    volatile float s1s2 = q.in_scale * q.f_scale;
    volatile float m1m2 = q.in_off * q.f_off;
    q.s1s2 = s1s2;
    q.m1 = q.in_off;
    q.m2 = q.f_off;
    q.m1m2 = m1m2;
    return q;
}

// One spatial dimension of TensorFlow's GetWindowedOutputSizeVerboseV2, which the
// reference calls at tf2/src/approx_nn_conv_ops.cpp:376-382.
static int window(int in, int k, int dil, int stride, int padding, int *out, int *pad_before)
{
    const long long eff = (long long)(k - 1) * dil + 1;
    if (padding == AXC_PADDING_VALID) {
        long long o = (in - eff + stride) / stride;
        if (in - eff + stride < 0) o = -1;
        *out = int(o);
        *pad_before = 0;
    } else {
        *out = (in + stride - 1) / stride;
        long long need = (long long)(*out - 1) * stride + eff - in;
        if (need < 0) need = 0;
        *pad_before = int(need / 2);
    }
    return *out < 0 ? AXC_INVALID_ARGUMENT : AXC_OK;
}

int resolve_geometry(const axc_conv_desc *d, bool depthwise, Geom *g)
{
    if (!d || !g) return AXC_INVALID_ARGUMENT;
    // Attribute checks of InitApproxConv2DParameters (tf2/src/approx_nn_conv_ops.cpp:254-309).
    if (d->data_format != AXC_FORMAT_NHWC && d->data_format != AXC_FORMAT_NCHW) return AXC_INVALID_ARGUMENT;
    if (d->stride_h <= 0 || d->stride_w <= 0) return AXC_INVALID_ARGUMENT;
    if (d->dil_h <= 0 || d->dil_w <= 0) return AXC_INVALID_ARGUMENT;
    if (d->padding != AXC_PADDING_SAME && d->padding != AXC_PADDING_VALID && d->padding != AXC_PADDING_EXPLICIT)
        return AXC_INVALID_ARGUMENT;
    // Shape checks of ComputeApproxConv2DDimensions (:311-404).
    if (d->n < 0 || d->h < 0 || d->w < 0 || d->c < 0) return AXC_INVALID_ARGUMENT;
    if (d->kh <= 0 || d->kw <= 0 || d->filter_c <= 0 || d->cout < 0) return AXC_INVALID_ARGUMENT;
    if (d->c % d->filter_c != 0) return AXC_INVALID_ARGUMENT;  // "input depth must be evenly divisible by filter depth"
    // Layout and grouping the kernels do not cover (:160-163, 224-232, 622-625).
    if (d->data_format != AXC_FORMAT_NHWC) return AXC_UNIMPLEMENTED;
    if (d->padding == AXC_PADDING_EXPLICIT) return AXC_UNIMPLEMENTED;
    if (d->c != d->filter_c) return AXC_UNIMPLEMENTED;  // grouped convolution
    if (d->accumulate != AXC_ACCUM_EXACT_I32 && d->accumulate != AXC_ACCUM_REFERENCE_F32) return AXC_INVALID_ARGUMENT;
    g->accum = d->accumulate;
    if (d->plan != AXC_PLAN_KEEP && d->plan != AXC_PLAN_NONE) return AXC_INVALID_ARGUMENT;
    g->plan = d->plan;
    g->ep = Epilogue{nullptr, nullptr, 0, 0};

    g->N = d->n; g->H = d->h; g->W = d->w; g->C = d->c;
    g->KH = d->kh; g->KW = d->kw; g->Cout = d->cout;
    g->sh = d->stride_h; g->sw = d->stride_w; g->dh = d->dil_h; g->dw = d->dil_w;
    int rc = window(d->h, d->kh, d->dil_h, d->stride_h, d->padding, &g->OH, &g->ph);
    if (rc) return rc;
    rc = window(d->w, d->kw, d->dil_w, d->stride_w, d->padding, &g->OW, &g->pw);
    if (rc) return rc;
    const long long k = depthwise ? (long long)d->kh * d->kw : (long long)d->kh * d->kw * d->c;
    // "Patch too large for buffer" (:120-121): the reference's im2col chunk holds 4 Mi elements.
    if (k > (16ll * 1024 * 1024) / (long long)sizeof(float)) return AXC_INVALID_ARGUMENT;
    g->K = int(k);
    g->M = (long long)d->n * g->OH * g->OW;
    const long long out_c = depthwise ? (long long)d->c * d->cout : d->cout;
    if ((long long)d->n * d->h * d->w * d->c >= (1ll << 40) || g->M * out_c >= (1ll << 40)) return AXC_INVALID_ARGUMENT;
    if (out_c > (1ll << 30)) return AXC_INVALID_ARGUMENT;
    return AXC_OK;
}

static size_t round256(size_t v) { return (v + 255) & ~size_t(255); }

Workspace dense_workspace(int K, int Cout)
{
    Workspace w;
    const size_t kq = size_t((K + 3) / 4);
    w.prog_bytes = round256(kq * size_t(Cout) * 16);
    w.sums_off = w.prog_bytes;
    w.status_off = w.sums_off + round256(size_t(Cout) * 4);
    w.total = w.status_off + 256;
    return w;
}

size_t dense_workspace_total(int K, int Cout, long long)
{
    return plan_layout(K, Cout).total + dense_workspace(K, Cout).total;
}

Workspace depthwise_workspace(int KHW, int C, int mult)
{
    Workspace w;
    const size_t oc = size_t(C) * size_t(mult);
    w.prog_bytes = round256((size_t(KHW) + size_t(KHW + 1) / 2) * oc * 4);   // program words + two-tap packed words
    w.sums_off = w.prog_bytes;
    w.status_off = w.sums_off + round256(oc * 4);
    w.total = w.status_off + 256;
    return w;
}

const uint16_t *table_device_ptr(axc_table *t, int device, int *status)
{
    *status = AXC_OK;
    std::lock_guard<std::mutex> lock(t->mu);
    if (device < 0) {
        *status = AXC_INVALID_ARGUMENT;
        return nullptr;
    }
    if (size_t(device) < t->dev.size() && t->dev[size_t(device)]) return t->dev[size_t(device)];
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) {
        *status = cuda_failed(e);
        return nullptr;
    }
    if (device >= count) {
        *status = AXC_INVALID_ARGUMENT;
        return nullptr;
    }
    int prev = 0;
    cudaGetDevice(&prev);
    uint16_t *p = nullptr;
    e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaMalloc(&p, 65536 * sizeof(uint16_t));
    if (e == cudaSuccess) e = cudaMemcpy(p, t->host.data(), 65536 * sizeof(uint16_t), cudaMemcpyHostToDevice);
    // A copy from pageable host memory returns once the data is staged; the transfer itself is ordered on the legacy
    // stream only.  The caller's stream may be a non-blocking one, which does not wait for the legacy stream: wait
    // here until the replica is complete (once per table and device).
    if (e == cudaSuccess) e = cudaStreamSynchronize(cudaStreamLegacy);
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        *status = cuda_failed(e);
        return nullptr;
    }
    if (t->dev.size() <= size_t(device)) t->dev.resize(size_t(device) + 1, nullptr);
    t->dev[size_t(device)] = p;
    return p;
}

const uint16_t *table_device_ptr_if_resident(axc_table *t, int device)
{
    std::lock_guard<std::mutex> lock(t->mu);
    if (device < 0 || size_t(device) >= t->dev.size()) return nullptr;
    return t->dev[size_t(device)];
}

__global__ void layout_probe_kernel(unsigned *out2)
{
    extern __shared__ __align__(16) unsigned char probe_smem[];
    unsigned size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(size));
    out2[0] = (unsigned)__cvta_generic_to_shared(probe_smem);
    out2[1] = out2[0] + size;
}
static __device__ unsigned g_layout_probe[2];

int device_info(int device, DeviceInfo *out)
{
    static std::mutex mu;
    static std::vector<DeviceInfo> cache;
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0) return AXC_INVALID_ARGUMENT;
    if (size_t(device) < cache.size() && cache[size_t(device)].sm_count > 0) {
        *out = cache[size_t(device)];
        return AXC_OK;
    }
    DeviceInfo di;
    AXC_CUDA(cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, device));
    AXC_CUDA(cudaDeviceGetAttribute(&di.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    {
        // where the dynamic shared memory of a CTA really starts and ends on this device and driver
        int prev = 0;
        AXC_CUDA(cudaGetDevice(&prev));
        if (prev != device) AXC_CUDA(cudaSetDevice(device));
        unsigned *sym = nullptr;
        unsigned host2[2] = {0, 0};
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&sym), g_layout_probe);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(layout_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin);
        if (e == cudaSuccess) {
            layout_probe_kernel<<<1, 1, size_t(di.max_smem_optin)>>>(sym);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpy(host2, sym, sizeof(host2), cudaMemcpyDeviceToHost);
        if (prev != device) cudaSetDevice(prev);
        if (e != cudaSuccess) return cuda_failed(e);
        di.smem_base = host2[0];
        di.smem_end = host2[1];
    }
    if (cache.size() <= size_t(device)) cache.resize(size_t(device) + 1, DeviceInfo{0, 0, 0, 0});
    cache[size_t(device)] = di;
    *out = di;
    return AXC_OK;
}

// Shared body of the two forward entry points.
static int forward(bool depthwise, axc_table *table, const axc_conv_desc *desc, const float *input,
                   const float *filter, const float *ranges_dev, float in_min, float in_max, float f_min, float f_max,
                   float *output, void *workspace, size_t workspace_bytes, const axc_debug_out *dbg,
                   int device, void *stream, const axc_epilogue *epilogue = nullptr)
{
    if (!table || !desc) return AXC_INVALID_ARGUMENT;
    Geom g;
    int rc = resolve_geometry(desc, depthwise, &g);
    if (rc) return rc;
    if (epilogue) g.ep = Epilogue{epilogue->bias, epilogue->residual, epilogue->relu != 0 ? 1 : 0, epilogue->input_relu != 0 ? 1 : 0};
    const long long out_c = depthwise ? (long long)g.C * g.Cout : g.Cout;
    if (g.M * out_c == 0) return AXC_OK;  // empty output: nothing to do
    if (!input || !filter || !output) return AXC_INVALID_ARGUMENT;
    const size_t ws_total = depthwise ? depthwise_workspace(g.K, g.C, g.Cout).total : dense_workspace_total(g.K, g.Cout, g.M);
    if (!workspace || workspace_bytes < ws_total) return AXC_INTERNAL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return AXC_INVALID_ARGUMENT;

    int status = AXC_OK;
    const uint16_t *lut = table_device_ptr(table, device, &status);
    if (status) return status;

    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    const Quant q = make_quant(in_min, in_max, f_min, f_max);
    // The reference's fp32 running total is served by the integer kernels whenever it provably equals the exact
    // sum; a sum that could overflow an int32 accumulator is always added up the reference's way.
    const bool ref_order = !depthwise && ((g.accum == AXC_ACCUM_REFERENCE_F32 && !table_sum_exact_in_fp32(table, g.K)) ||
                                          !table_sum_fits_int32(table, g.K));
    rc = depthwise ? launch_depthwise(lut, g, q, input, filter, output, workspace, dbg, device, cudaStream_t(stream))
                   : launch_dense(lut, table_uid(table), g, q, ranges_dev, input, filter, output, workspace, dbg, device,
                                  cudaStream_t(stream), ref_order);
    if (prev != device) cudaSetDevice(prev);
    return rc;
}

}  // namespace axc

extern "C" {

int axc_table_create_from_memory(const uint16_t *lut65536, axc_table **out)
{
    if (!lut65536 || !out) return AXC_INVALID_ARGUMENT;
    axc_table *t = new (std::nothrow) axc_table;
    if (!t) return AXC_INTERNAL;
    t->host.assign(lut65536, lut65536 + 65536);
    axc::stamp(t);
    *out = t;
    return AXC_OK;
}

int axc_table_create_exact(axc_table **out)
{
    if (!out) return AXC_INVALID_ARGUMENT;
    axc_table *t = new (std::nothrow) axc_table;
    if (!t) return AXC_INTERNAL;
    t->host.resize(65536);
    for (uint32_t i = 0; i < 65536u; ++i) t->host[i] = uint16_t((i >> 8) * (i & 0xFFu));
    axc::stamp(t);
    *out = t;
    return AXC_OK;
}

int axc_table_create_from_file(const char *path, int num_bits, axc_table **out)
{
    if (!out) return AXC_INVALID_ARGUMENT;
    // The table index shift and the exact-product fallback of the reference only work
    // for 8 bits (tf2/src/approx_ops_types.h:110-117).
    if (num_bits != 8) return AXC_INVALID_ARGUMENT;
    if (!path || !path[0]) return axc_table_create_exact(out);
    FILE *f = std::fopen(path, "rb");
    if (!f) return AXC_INVALID_ARGUMENT;
    axc_table *t = new (std::nothrow) axc_table;
    if (!t) {
        std::fclose(f);
        return AXC_INTERNAL;
    }
    t->host.assign(65536, 0);
    const size_t got = std::fread(t->host.data(), sizeof(uint16_t), 65536, f);
    std::fclose(f);
    if (got != 65536) {
        delete t;
        return AXC_INVALID_ARGUMENT;
    }
    axc::stamp(t);
    *out = t;
    return AXC_OK;
}

void axc_table_destroy(axc_table *t)
{
    if (!t) return;
    int prev = 0;
    cudaGetDevice(&prev);
    for (size_t d = 0; d < t->dev.size(); ++d)
        if (t->dev[d]) {
            cudaSetDevice(int(d));
            cudaFree(t->dev[d]);
        }
    cudaSetDevice(prev);
    delete t;
}

// Weight tuning of the first-generation op (tf1/axqconv/approximate_selector.h:46-78): per weight w the column
// that is closest to the exact products in summed absolute error stands in for column w.
int axc_table_tune_weights(const uint16_t *in, uint16_t *out)
{
    if (!in || !out) return AXC_INVALID_ARGUMENT;
    // err[w][w2] = sum_i |i*w - in[i][w2]| is needed for all pairs; walk i outermost so that rows stream
    std::vector<int> err(256 * 256, 0);
    for (int i = 0; i < 256; ++i) {
        const uint16_t *row = in + i * 256;
        for (int w = 0; w < 256; ++w) {
            const int exact = i * w;
            int *e = err.data() + w * 256;
            for (int w2 = 0; w2 < 256; ++w2) {
                const int d = exact - int(row[w2]);
                e[w2] += d < 0 ? -d : d;
            }
        }
    }
    int map[256];
    for (int w = 0; w < 256; ++w) {
        const int *e = err.data() + w * 256;
        int best = 0;
        for (int w2 = 1; w2 < 256; ++w2)
            if (e[w2] < e[best]) best = w2;
        map[w] = e[w] == e[best] ? w : best;      // w itself among the best columns wins, else the lowest index
    }
    std::vector<uint16_t> tmp(in, in + 65536);    // `in` and `out` may alias
    for (int i = 0; i < 256; ++i)
        for (int w = 0; w < 256; ++w) out[i * 256 + w] = tmp[i * 256 + map[w]];
    return AXC_OK;
}

int axc_table_host_data(const axc_table *t, const uint16_t **out)
{
    if (!t || !out) return AXC_INVALID_ARGUMENT;
    *out = t->host.data();
    return AXC_OK;
}

int axc_table_ensure_device(axc_table *t, int device)
{
    if (!t) return AXC_INVALID_ARGUMENT;
    int status = AXC_OK;
    axc::table_device_ptr(t, device, &status);
    if (status) return status;
    axc::DeviceInfo di;
    return axc::device_info(device, &di);     // the one-time shared-memory probe of the device happens here, too
}

int axc_conv2d_output_dims(const axc_conv_desc *desc, int64_t out4[4])
{
    if (!out4) return AXC_INVALID_ARGUMENT;
    axc::Geom g;
    int rc = axc::resolve_geometry(desc, false, &g);
    if (rc) return rc;
    out4[0] = g.N; out4[1] = g.OH; out4[2] = g.OW; out4[3] = g.Cout;
    return AXC_OK;
}

int axc_depthwise_conv2d_output_dims(const axc_conv_desc *desc, int64_t out4[4])
{
    if (!out4) return AXC_INVALID_ARGUMENT;
    axc::Geom g;
    int rc = axc::resolve_geometry(desc, true, &g);
    if (rc) return rc;
    out4[0] = g.N; out4[1] = g.OH; out4[2] = g.OW; out4[3] = int64_t(g.C) * g.Cout;
    return AXC_OK;
}

int axc_conv2d_workspace_bytes(const axc_conv_desc *desc, size_t *bytes)
{
    if (!bytes) return AXC_INVALID_ARGUMENT;
    axc::Geom g;
    int rc = axc::resolve_geometry(desc, false, &g);
    if (rc) return rc;
    *bytes = axc::dense_workspace_total(g.K, g.Cout, g.M);
    return AXC_OK;
}

int axc_depthwise_conv2d_workspace_bytes(const axc_conv_desc *desc, size_t *bytes)
{
    if (!bytes) return AXC_INVALID_ARGUMENT;
    axc::Geom g;
    int rc = axc::resolve_geometry(desc, true, &g);
    if (rc) return rc;
    *bytes = axc::depthwise_workspace(g.K, g.C, g.Cout).total;
    return AXC_OK;
}

int axc_conv2d_forward(axc_table *table, const axc_conv_desc *desc, const float *input, const float *filter,
                       float in_min, float in_max, float f_min, float f_max, float *output,
                       void *workspace, size_t workspace_bytes, const axc_debug_out *debug, int device,
                       void *stream)
{
    return axc::forward(false, table, desc, input, filter, nullptr, in_min, in_max, f_min, f_max, output, workspace,
                        workspace_bytes, debug, device, stream);
}

int axc_conv2d_forward_fused(axc_table *table, const axc_conv_desc *desc, const float *input, const float *filter,
                             float in_min, float in_max, float f_min, float f_max, const float *ranges,
                             const axc_epilogue *epilogue, float *output, void *workspace, size_t workspace_bytes,
                             const axc_debug_out *debug, int device, void *stream)
{
    return axc::forward(false, table, desc, input, filter, ranges, in_min, in_max, f_min, f_max, output, workspace,
                        workspace_bytes, debug, device, stream, epilogue);
}

int axc_depthwise_conv2d_forward_fused(axc_table *table, const axc_conv_desc *desc, const float *input,
                                       const float *filter, float in_min, float in_max, float f_min, float f_max,
                                       const axc_epilogue *epilogue, float *output, void *workspace,
                                       size_t workspace_bytes, const axc_debug_out *debug, int device, void *stream)
{
    return axc::forward(true, table, desc, input, filter, nullptr, in_min, in_max, f_min, f_max, output, workspace,
                        workspace_bytes, debug, device, stream, epilogue);
}

int axc_conv2d_forward_device_ranges(axc_table *table, const axc_conv_desc *desc, const float *input,
                                     const float *filter, const float *ranges, float *output, void *workspace,
                                     size_t workspace_bytes, const axc_debug_out *debug, int device, void *stream)
{
    if (!ranges) return AXC_INVALID_ARGUMENT;
    return axc::forward(false, table, desc, input, filter, ranges, 0.f, 0.f, 0.f, 0.f, output, workspace,
                        workspace_bytes, debug, device, stream);
}

int axc_conv2d_forward_sharded(axc_table *table, const axc_conv_desc *desc, const axc_shard *shards, int32_t nshards,
                               float in_min, float in_max, float f_min, float f_max, int32_t *failed_shard)
{
    if (failed_shard) *failed_shard = -1;
    if (!table || !desc || !shards || nshards <= 0) return AXC_INVALID_ARGUMENT;
    for (int32_t i = 0; i < nshards; ++i) {
        const axc_shard &sh = shards[i];
        axc_conv_desc d = *desc;
        d.n = sh.n;
        const int rc = axc::forward(false, table, &d, sh.input, sh.filter, nullptr, in_min, in_max, f_min, f_max, sh.output,
                                    sh.workspace, sh.workspace_bytes, nullptr, sh.device, sh.stream);
        if (rc != AXC_OK) {
            if (failed_shard) *failed_shard = i;
            return rc;
        }
    }
    return AXC_OK;
}

int axc_gather_outputs(const axc_shard *shards, int32_t nshards, size_t image_bytes, void *dst, int32_t dst_device)
{
    if (!shards || nshards <= 0 || !dst) return AXC_INVALID_ARGUMENT;
    unsigned char *p = static_cast<unsigned char *>(dst);
    for (int32_t i = 0; i < nshards; ++i) {
        const axc_shard &sh = shards[i];
        const size_t bytes = size_t(sh.n) * image_bytes;
        if (bytes > 0) {
            if (!sh.output) return AXC_INVALID_ARGUMENT;
            AXC_CUDA(cudaMemcpyPeerAsync(p, dst_device, sh.output, sh.device, bytes, cudaStream_t(sh.stream)));
        }
        p += bytes;
    }
    return AXC_OK;
}

int axc_depthwise_conv2d_forward(axc_table *table, const axc_conv_desc *desc, const float *input,
                                 const float *filter, float in_min, float in_max, float f_min, float f_max,
                                 float *output, void *workspace, size_t workspace_bytes,
                                 const axc_debug_out *debug, int device, void *stream)
{
    return axc::forward(true, table, desc, input, filter, nullptr, in_min, in_max, f_min, f_max, output, workspace,
                        workspace_bytes, debug, device, stream);
}

int axc_conv2d_plan_info(const void *workspace, int32_t out4[4], int device, void *stream)
{
    if (!workspace || !out4) return AXC_INVALID_ARGUMENT;
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    const int rc = axc::plan_info(workspace, out4, cudaStream_t(stream));
    if (prev != device) cudaSetDevice(prev);
    return rc;
}

int axc_depthwise_conv2d_status(const axc_conv_desc *desc, const void *workspace, int32_t *status, int device, void *stream)
{
    if (!status) return AXC_INVALID_ARGUMENT;
    axc::Geom g;
    int rc = axc::resolve_geometry(desc, true, &g);
    if (rc) return rc;
    return axc::depthwise_status(g, workspace, status, device, cudaStream_t(stream));
}

int axc_debug_bounds_record(int device, uint32_t out4[4])
{
    if (!out4) return AXC_INVALID_ARGUMENT;
#ifndef AXC_BOUNDS_CHECK
    (void)device;
    out4[0] = out4[1] = out4[2] = out4[3] = 0;
    return AXC_UNIMPLEMENTED;
#else
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    cudaError_t e = cudaDeviceSynchronize();
    unsigned parts[3][4] = {};
    int rc = e == cudaSuccess ? AXC_OK : axc::cuda_failed(e);
    if (rc == AXC_OK) rc = axc::bounds_record_sched(parts[0]);
    if (rc == AXC_OK) rc = axc::bounds_record_conv(parts[1]);
    if (rc == AXC_OK) rc = axc::bounds_record_depthwise(parts[2]);
    if (prev != device) cudaSetDevice(prev);
    out4[0] = out4[1] = out4[2] = out4[3] = 0;
    for (int t = 0; t < 3; ++t) {
        if (parts[t][0] != 0 && out4[0] == 0) { out4[1] = parts[t][1]; out4[2] = parts[t][2]; out4[3] = parts[t][3]; }
        out4[0] += parts[t][0];
    }
    return rc;
#endif
}

int axc_quant_props(float min_value, float max_value, float out3[3])
{
    if (!out3) return AXC_INVALID_ARGUMENT;
    axc::var_quant_props(min_value, max_value, &out3[0], &out3[1], &out3[2]);
    return AXC_OK;
}

const char *axc_status_string(int status)
{
    switch (status) {
    case AXC_OK: return "OK";
    case AXC_INVALID_ARGUMENT: return "InvalidArgument";
    case AXC_UNIMPLEMENTED: return "Unimplemented";
    case AXC_INTERNAL: return "Internal";
    case AXC_CUDA_ERROR: return "CudaError";
    default: return "Unknown";
    }
}

int axc_last_cuda_error(void) { return axc::g_last_cuda_error; }

uint64_t axc_launch_count(void) { return axc::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
