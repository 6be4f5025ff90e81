// Measurement of the shared-memory lookup peak: what one SM sustains in conflict-free 16-bit shared-memory loads,
// the operation every table MAC of the dense kernels costs.  The roofline of those kernels is quoted against
// 32 lookups per clock and SM by construction of the hardware (32 banks, one wavefront per clock); this kernel
// measures that figure on the device at hand, so that the fraction has a measured denominator as well.
#include <vector>

#include "axc_internal.h"

namespace axc {

namespace {

constexpr int kProbeThreads = 512;
constexpr int kProbeUnroll = 16;
constexpr int kProbeIters = 4096;

// Every lane reads its own bank (conflict-free); the address of a load depends on the value of an earlier one
// through a mask that is zero at run time, so the loads can neither be hoisted nor merged.
__global__ void __launch_bounds__(kProbeThreads, 1) lookup_peak_kernel(const unsigned *zero_mask, long long *cycles, unsigned *sink)
{
    __shared__ __align__(16) unsigned table[8192];            // 32 KiB
    for (int i = threadIdx.x; i < 8192; i += kProbeThreads) table[i] = unsigned(i) * 2654435761u;
    const unsigned mask = *zero_mask;
    __syncthreads();
    const unsigned lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const unsigned base = (unsigned)__cvta_generic_to_shared(table) + lane * 4u + (warp & 7u) * 128u;
    unsigned acc[kProbeUnroll];
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) acc[u] = 0;
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < kProbeIters; ++it) {
#pragma unroll
        for (int u = 0; u < kProbeUnroll; ++u) {
            unsigned v;
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(base + unsigned(u) * 1024u + (acc[u] & mask)));
            acc[u] = v;
        }
    }
    __syncthreads();
    const long long t1 = clock64();
    if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
    unsigned x = 0;
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) x ^= acc[u];
    if (x == 0xFFFFFFFFu) sink[0] = x;                        // keeps the loads alive
}

}  // namespace

}  // namespace axc

extern "C" int axc_measure_lookup_peak(int device, void *scratch, size_t scratch_bytes, void *stream,
                                       double *lookups_per_clk_per_sm)
{
    using namespace axc;
    if (!scratch || !lookups_per_clk_per_sm) return AXC_INVALID_ARGUMENT;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    const size_t need = 256 + size_t(di.sm_count) * sizeof(long long);
    if (scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return AXC_INVALID_ARGUMENT;
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    cudaStream_t s = cudaStream_t(stream);
    unsigned char *b = static_cast<unsigned char *>(scratch);
    cudaError_t e = cudaMemsetAsync(b, 0, need, s);
    std::vector<long long> cyc(size_t(di.sm_count), 0);
    if (e == cudaSuccess) {
        lookup_peak_kernel<<<unsigned(di.sm_count), kProbeThreads, 0, s>>>(reinterpret_cast<unsigned *>(b), reinterpret_cast<long long *>(b + 256),
                                                                           reinterpret_cast<unsigned *>(b + 128));
        e = cudaGetLastError();
        count_launch();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(cyc.data(), b + 256, cyc.size() * sizeof(long long), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_failed(e);
    long long worst = 1;
    for (long long c : cyc) worst = c > worst ? c : worst;
    *lookups_per_clk_per_sm = double(kProbeThreads) * kProbeUnroll * kProbeIters / double(worst);
    return AXC_OK;
}
