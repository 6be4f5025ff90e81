// Internal declarations shared by the translation units of libaxconv.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "axconv.h"

// ---- debug flavour with bounds checks (-DAXC_BOUNDS_CHECK, libaxconv_check.so) ---------------------------------
// Every shared-memory address the kernels compute and every global index they form from the launch parameters is
// checked before use.  A violation is counted, the first one is recorded (site number and offending value) and the
// access is skipped (loads give 0): the kernel finishes, nothing traps, and axc_debug_bounds_record() reports.  In the
// normal build the macros are `true` and cost nothing.
#ifdef AXC_BOUNDS_CHECK
namespace axc {
// one record per translation unit (the library is built without relocatable device code):
// {violations, site of the first, its value low word, high word}
static __device__ unsigned g_bounds_record[4];
__device__ __forceinline__ bool bounds_note(bool ok, unsigned site, unsigned long long value)
{
    if (!ok && atomicAdd(&g_bounds_record[0], 1u) == 0u) {
        g_bounds_record[1] = site;
        g_bounds_record[2] = unsigned(value);
        g_bounds_record[3] = unsigned(value >> 32);
    }
    return ok;
}
// `bytes` (a power of two) at the shared-window address `addr`: inside [lo, hi) and aligned
__device__ __forceinline__ bool shared_ok(unsigned addr, unsigned bytes, unsigned lo, unsigned hi, unsigned site)
{
    unsigned window;
    asm("mov.u32 %0, %%aggr_smem_size;" : "=r"(window));      // user + reserved shared memory of this CTA
    hi = hi < window ? hi : window;
    return bounds_note(addr >= lo && addr + bytes <= hi && (addr & (bytes - 1u)) == 0u, site, addr);
}
__device__ __forceinline__ bool global_ok(long long index, long long count, unsigned site)
{
    return bounds_note(index >= 0 && index < count, site, (unsigned long long)index);
}
}  // namespace axc
#define AXC_SHARED_OK(addr, bytes, lo, hi, site) (::axc::shared_ok((addr), (bytes), (lo), (hi), (site)))
#define AXC_GLOBAL_OK(index, count, site) (::axc::global_ok((index), (count), (site)))
#else
#define AXC_SHARED_OK(addr, bytes, lo, hi, site) (true)
#define AXC_GLOBAL_OK(index, count, site) (true)
#endif

namespace axc {

// Reads and clears this translation unit's bounds record (all zeros in the normal build).  Defined once per .cu file
// that has checked kernels, under its own name.
#ifdef AXC_BOUNDS_CHECK
#define AXC_DEFINE_BOUNDS_READER(name)                                                                   \
    int name(unsigned out4[4])                                                                           \
    {                                                                                                    \
        const unsigned zero[4] = {0, 0, 0, 0};                                                           \
        AXC_CUDA(cudaMemcpyFromSymbol(out4, g_bounds_record, sizeof(zero)));                             \
        AXC_CUDA(cudaMemcpyToSymbol(g_bounds_record, zero, sizeof(zero)));                               \
        return AXC_OK;                                                                                   \
    }
#else
#define AXC_DEFINE_BOUNDS_READER(name)                \
    int name(unsigned out4[4])                        \
    {                                                 \
        out4[0] = out4[1] = out4[2] = out4[3] = 0;    \
        return AXC_OK;                                \
    }
#endif
int bounds_record_sched(unsigned out4[4]);
int bounds_record_conv(unsigned out4[4]);
int bounds_record_depthwise(unsigned out4[4]);

// Quantisation state of one call: what the reference keeps in
// BaseTableApproxOpType_t::quantProps (tf2/src/approx_ops_types.h:84-96).
struct Quant {
    float in_scale, in_inv, in_off;
    float f_scale, f_inv, f_off;
    float s1s2, m1, m2, m1m2;
};

// Optional additions fused into the dequantisation (axc_epilogue of the C ABI).
struct Epilogue {
    const float *bias;      // [out channels] or NULL
    const float *residual;  // output shape or NULL
    int relu;
    int input_relu;         // max(x, 0) on every input element as it is loaded (the producer's ReLU, applied here)
};

// y after the fused epilogue; `idx` = element index of the output, `bias_j` = bias of its channel (0 without one)
__device__ __forceinline__ float apply_epilogue(float y, const Epilogue &ep, float bias_j, long long idx)
{
    if (ep.bias) y = __fadd_rn(y, bias_j);
    if (ep.residual) y = __fadd_rn(y, __ldg(ep.residual + idx));
    if (ep.relu) y = fmaxf(y, 0.0f);
    return y;
}

// max(y, floor) that keeps a NaN: the fused ReLU is this with floor = 0, no ReLU is floor = -inf - one instruction
// either way, no branch and no select in the kernels' epilogues.
__device__ __forceinline__ float max_keep_nan(float y, float floor)
{
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(y), "f"(floor));
    return d;
}

// Resolved geometry (TensorFlow window arithmetic applied).
struct Geom {
    int N, H, W, C;
    int KH, KW, Cout;  // depthwise: Cout = channel multiplier
    int sh, sw, dh, dw;
    int ph, pw;        // padding before (rows, cols)
    int OH, OW;
    int K;             // dense: KH*KW*C; depthwise: KH*KW
    long long M;       // N*OH*OW
    int accum;         // AXC_ACCUM_*
    int plan;          // AXC_PLAN_*
    Epilogue ep;       // set by the entry point after resolve_geometry
};

void var_quant_props(float min_v, float max_v, float *scale, float *inv, float *offset);
Quant make_quant(float in_min, float in_max, float f_min, float f_max);

// Validates `d` the way the reference op does and fills `g`.  depthwise selects the
// grouped interpretation of the filter.
int resolve_geometry(const axc_conv_desc *d, bool depthwise, Geom *g);

// Records a failed CUDA call for axc_last_cuda_error() and returns AXC_CUDA_ERROR.
int cuda_failed(cudaError_t e);
void count_launch(int n = 1);

#define AXC_CUDA(expr)                                        \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) return ::axc::cuda_failed(_e); \
    } while (0)

// Device replica of a table (native [a][b] order, 65536 uint16).
const uint16_t *table_device_ptr(axc_table *t, int device, int *status);
// The replica on `device` if it has been uploaded already, else NULL.  Never allocates.
const uint16_t *table_device_ptr_if_resident(axc_table *t, int device);
// Process-unique id of a table handle (tables are immutable after creation).
unsigned table_uid(const axc_table *t);
// True when a sum of K entries of the table, added one by one in fp32 in any order, cannot round: every partial
// sum is a multiple of 2^tz (tz = trailing zero bits common to all entries) and at most K * largest entry, and
// fp32 holds every such multiple up to 2^(24 + tz).
bool table_sum_exact_in_fp32(const axc_table *t, long long K);
// True when K entries cannot overflow an int32 accumulator.
bool table_sum_fits_int32(const axc_table *t, long long K);

struct DeviceInfo {
    int sm_count;
    int max_smem_optin;
    // Shared-memory window of a CTA launched with max_smem_optin bytes of dynamic shared memory, as a probe kernel
    // saw it on this device: address of the first dynamic byte and the byte after the last.  The dense kernels place
    // the table planes at fixed window addresses (64 KiB and 128 KiB) and need the window to reach 228 KiB.
    unsigned smem_base, smem_end;
};
// Attributes of `device` (cached).  The first call for a device launches a one-thread probe kernel and waits for it.
int device_info(int device, DeviceInfo *out);
// Status word of the depthwise scratch of this shape (0 = fine); workspace == NULL: the built-in scratch.
int depthwise_status(const Geom &g, const void *workspace, int32_t *status, int device, cudaStream_t stream);

// ---- workspace layout (dense) ---------------------------------------------------------
//   [0, prog_bytes)            kernel-layout filter program: uint4 per (l/4, j)
//   [prog_bytes, +4*Cout)      per-channel fp32 filter sums
//   [.., +16)                  status word (0 = fine)
struct Workspace {
    size_t prog_bytes, sums_off, status_off, total;
};
Workspace dense_workspace(int K, int Cout);      // region of the common-K kernel
size_t dense_workspace_total(int K, int Cout, long long M);   // plan of the scheduled kernel + that region (M unused)
Workspace depthwise_workspace(int KHW, int C, int mult);

// Kernel launchers (axc_conv.cu / axc_depthwise.cu).
// ranges_dev: NULL, or {in_min, in_max, f_min, f_max} in device memory (then `q` is ignored).
// ref_order: add the products up in K order with an fp32 running total (the reference's arithmetic) instead of
// the exact integer sum.
int launch_dense(const uint16_t *lut_dev, unsigned table_uid, const Geom &g, const Quant &q, const float *ranges_dev,
                 const float *input, const float *filter, float *output, void *workspace, const axc_debug_out *dbg,
                 int device, cudaStream_t stream, bool ref_order);
// out = out (+ bias[channel]) (+ residual), then max(out, 0) if relu, in one pass; bias / residual may be NULL
int launch_post(float *out, const float *bias, const float *residual, long long count, int channels, int relu,
                const DeviceInfo &di, cudaStream_t stream);
int launch_depthwise(const uint16_t *lut_dev, const Geom &g, const Quant &q, const float *input,
                     const float *filter, float *output, void *workspace, const axc_debug_out *dbg,
                     int device, cudaStream_t stream);

}  // namespace axc
