// Dense table-driven convolution for sm_100a: one persistent kernel that fuses the
// activation quantiser, the patch gather (im2col), the table GEMM with int32 accumulators
// and the fp32 dequantisation, plus two small filter-preparation kernels.
//
// It replaces the reference's per-chunk sequence im2col kernel -> GEMM kernel
// (tf2/src/cuda/approx_nn_conv_kernels.cu:415-489, 513-625) and its broken fused 1x1 kernel
// (:323-394); the arithmetic follows the reference's CPU kernels
// (tf2/src/approx_nn_conv_kernels.cpp:167-296).
//
// Shared-memory plan of the main kernel (addresses in the CTA's shared window):
//   [dyn0, 65536)        staging: activation tiles, filter-program tiles, pixel table
//   [65536, 131072)      table plane 0: entries with weight b < 128,  byte a*256 + 2*b
//   [131072, 196608)     table plane 1: entries with weight b >= 128, byte a*256 + 2*(b-128)
//   [196608, 196624)     a zero word, target of the K-tail padding
// With the planes on 64 KiB boundaries the byte address of LUT[a][b] is the four bytes
// {2*(b&127), a, 1+(b>>7), 0}: one PRMT builds it from the filter-program word
// {2*(b&127), 0, 1+(b>>7), 0} and a packed activation word, so a table MAC costs
// PRMT + LDS.U16 + IADD.
#include <cstdio>
#include <cstdlib>

#include <cmath>

#include "axc_internal.h"
#include "axc_sched.h"

namespace axc {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPixPerLane = 16;       // output pixels accumulated by one lane
constexpr int kKC = 64;               // K elements per staged chunk
constexpr int kLQ = kKC / 4;          // quads of K per chunk
constexpr unsigned kLutBase = 65536u;
constexpr unsigned kZeroWordAddr = 196608u;
constexpr unsigned kSmemEnd = kZeroWordAddr + 16u;
constexpr uint32_t kProgPadK = 0x00030000u;   // -> address kZeroWordAddr when the activation byte is 0
constexpr uint32_t kProgPadN = 0x00010000u;   // any valid table address; result is never stored

struct DenseParams {
    const uint16_t *lut;
    const float *input;
    float *output;
    const uint4 *prog;     // [ceil(K/4)][Cout] filter-program quads
    const float *bsum;     // [Cout]
    int32_t *acc_out;      // optional [M][Cout]
    int *status;
    int N, H, W, C, KH, KW, Cout;
    int sh, sw, dh, dw, ph, pw, OH, OW, K;
    long long M;
    int tiles_n;
    long long tiles_total;
    const DevQuant *dq;    // quantisation parameters of the call (workspace header)
    int vec_ok;            // C % 4 == 0 and 16-byte aligned input
    const int *gate;       // when set: run only if *gate != 0 (the scheduled kernel handed the call over)
    float in_floor;        // every input element is max(x, in_floor) as it is loaded: 0 = the producer's ReLU, -inf = none
};

__device__ __forceinline__ unsigned quantize_u8(float x, float off, float inv)
{
    // uint8((x - off) * inv + 0.5f): three separately rounded operations
    // (tf2/src/approx_nn_conv_kernels.cpp:293), saturated to [0, 255].
    const float v = __fadd_rn(__fmul_rn(__fsub_rn(x, off), inv), 0.5f);
    const unsigned u = __float2uint_rz(v);  // negative and NaN -> 0
    return u > 255u ? 255u : u;
}

// Shared-memory accessors; the debug flavour checks every address first (table lookups: planes and zero word).
__device__ __forceinline__ unsigned lds_u16(unsigned addr)
{
    if (!AXC_SHARED_OK(addr, 2u, kLutBase, kSmemEnd, 201u)) return 0u;
    unsigned v;
    asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 lds_v4(unsigned addr)
{
    if (!AXC_SHARED_OK(addr, 16u, 0u, kSmemEnd, 202u)) return make_uint4(0, 0, 0, 0);
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts_u32(unsigned addr, unsigned v)
{
    if (!AXC_SHARED_OK(addr, 4u, 0u, kSmemEnd, 203u)) return;
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ void sts_v4(unsigned addr, uint4 v)
{
    if (!AXC_SHARED_OK(addr, 16u, 0u, kSmemEnd, 204u)) return;
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void sts_f32(unsigned addr, float v)
{
    if (!AXC_SHARED_OK(addr, 4u, 0u, kSmemEnd, 205u)) return;
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ float lds_f32(unsigned addr)
{
    if (!AXC_SHARED_OK(addr, 4u, 0u, kSmemEnd, 206u)) return 0.0f;
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// Filter preparation: quantise the fp32 filter [K][Cout] into kernel-layout program words
// (one uint4 per (l/4, j): the four words of l = 4*lq .. 4*lq+3) and, optionally, the plain
// uint8 matrix.  Weight quantiser as tf2/src/approx_nn_conv_kernels.cpp:243.
__global__ void filter_prep_kernel(const float *__restrict__ filter, int K, int Cout, const DevQuant *__restrict__ dq,
                                   uint4 *__restrict__ prog, uint8_t *__restrict__ qfilter, int *status,
                                   const int *gate)
{
    if (gate && *gate == 0) return;
    const float f_off = dq->f_off, f_inv = dq->f_inv;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx == 0) *status = 0;
    const int kq = (K + 3) / 4;
    if (idx >= (long long)kq * Cout) return;
    const int lq = int(idx / Cout), j = int(idx % Cout);
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int l = lq * 4 + e;
        if (l < K) {
            const unsigned b = quantize_u8(filter[(size_t)l * Cout + j], f_off, f_inv);
            w[e] = ((b & 127u) << 1) | ((1u + (b >> 7)) << 16);
            if (qfilter) qfilter[(size_t)l * Cout + j] = uint8_t(b);
        } else {
            w[e] = kProgPadK;
        }
    }
    prog[idx] = make_uint4(w[0], w[1], w[2], w[3]);
}

// Per output channel fp32 sum of the filter over (kh, kw, c), added in l order like the
// reference's fused form (tf2/src/approx_nn_conv_kernels.cpp:187-197; the Eigen reduction of
// :300-306 leaves the order open).  One thread per channel; loads are batched, adds are serial.
__global__ void filter_sum_kernel(const float *__restrict__ filter, int K, int Cout, float *__restrict__ bsum,
                                  const int *gate)
{
    if (gate && *gate == 0) return;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= Cout) return;
    float acc = 0.0f;
    int l = 0;
    for (; l + 8 <= K; l += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __ldg(filter + (size_t)(l + e) * Cout + j);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc = __fadd_rn(acc, v[e]);
    }
    for (; l < K; ++l) acc = __fadd_rn(acc, __ldg(filter + (size_t)l * Cout + j));
    bsum[j] = acc;
}

// Element-wise quantised copy of the input, for the parity taps only.
__global__ void quantize_tensor_kernel(const float *__restrict__ x, long long n, const DevQuant *__restrict__ dq,
                                       uint8_t *__restrict__ q, float in_floor)
{
    const float off = dq->in_off, inv = dq->in_inv;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) q[i] = uint8_t(quantize_u8(max_keep_nan(x[i], in_floor), off, inv));
}

// The table entry `v` (0..65535) as fp32 without a conversion instruction: 2^23 + v is exact in fp32 and has the
// bit pattern 0x4B000000 | v; subtracting 2^23 again is exact too.
__device__ __forceinline__ float entry_to_float(unsigned v)
{
    return __fsub_rn(__uint_as_float(0x4B000000u | v), 8388608.0f);
}

// One CTA per SM, persistent over output tiles of TM pixels x TN channels
// (TN = 32 * WN, TM = 16 * (8 / WN)).  Lane = output channel, 16 pixels per lane.
// REF = false: exact int32 sum.  REF = true: the reference's arithmetic, an fp32 running total that takes the
// entries one by one in K order (tf2/src/approx_nn_conv_kernels.cpp:245-246, 201-202); every lane walks K from
// 0 upwards, chunk by chunk, so the additions - and their roundings once the total passes 2^24 - are the
// reference's.
template <int WN, bool REF>
__global__ void __launch_bounds__(kThreads, 1) dense_kernel(const DenseParams P)
{
    constexpr int WM = kWarps / WN;
    constexpr int TM = WM * kPixPerLane;
    constexpr int TN = WN * 32;
    constexpr int AROW = TM + 4;                       // words per K-quad row of the activation tile
    constexpr int A_BYTES = kLQ * AROW * 4;
    constexpr int W_BYTES = kLQ * TN * 16;
    constexpr int PIX_SLOTS = (TM / 4) / kWarps;       // pixel groups a loader thread visits per K-quad half
    constexpr int A_ITERS = (kLQ / 8) * PIX_SLOTS;     // activation quads per thread per chunk
    constexpr int W_ITERS = (kLQ * TN) / kThreads;     // program quads per thread per chunk
    constexpr int SUM_WARPS = TM / 32;                 // warps that carry the patch sums of one chunk
    constexpr int SUM_GROUPS = kWarps / SUM_WARPS;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (P.gate && *P.gate == 0) return;
    const DevQuant Q = *P.dq;
    const unsigned dyn0 = (unsigned)__cvta_generic_to_shared(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // staging layout, from the first 16-byte boundary at or after dyn0
    unsigned cur = (dyn0 + 15u) & ~15u;
    const unsigned sA = cur;            cur += 2 * A_BYTES;
    const unsigned sW = cur;            cur += 2 * W_BYTES;
    const unsigned sPixBase = cur;      cur += TM * 8;   // long long element offset of (n, iy0, ix0, 0)
    const unsigned sPixY = cur;         cur += TM * 4;
    const unsigned sPixX = cur;         cur += TM * 4;
    const unsigned sAsum = cur;         cur += TM * 4;
    unsigned dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (cur > kLutBase || dyn0 + dyn_size < kSmemEnd) {
        if (tid == 0) atomicExch(P.status, 1);
        return;
    }

    // ---- table planes --------------------------------------------------------------
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(P.lut);
        for (int i = tid; i < 8192; i += kThreads) {
            const int a = i >> 5, part = i & 31;
            const uint4 v = __ldg(src + i);
            const unsigned dst = kLutBase + (part >= 16 ? 65536u : 0u) + unsigned(a) * 256u + unsigned(part & 15) * 16u;
            sts_v4(dst, v);
        }
        if (tid == 0) sts_v4(kZeroWordAddr, make_uint4(0, 0, 0, 0));
    }

    const int wn = warp % WN, wm = warp / WN;
    const int lq_lo = lane & 7, p_lo = lane >> 3;

    for (long long tile = blockIdx.x; tile < P.tiles_total; tile += gridDim.x) {
        const long long mt = tile / P.tiles_n;
        const int nt = int(tile - mt * P.tiles_n);
        const long long m0 = mt * TM;
        const int j0 = nt * TN;

        __syncthreads();  // previous tile fully consumed (also orders the table fill)
        if (tid < TM) {
            const long long p = m0 + tid;
            long long base = 0;
            int iy0 = -(1 << 28), ix0 = -(1 << 28);  // invalid pixel: every tap out of range
            if (p < P.M) {
                const int ow = int(p % P.OW);
                const long long t = p / P.OW;
                const int oh = int(t % P.OH);
                const int n = int(t / P.OH);
                iy0 = oh * P.sh - P.ph;
                ix0 = ow * P.sw - P.pw;
                base = (((long long)n * P.H + iy0) * P.W + ix0) * P.C;
            }
            asm volatile("st.shared.u64 [%0], %1;" ::"r"(sPixBase + tid * 8), "l"(base) : "memory");
            sts_u32(sPixY + tid * 4, unsigned(iy0));
            sts_u32(sPixX + tid * 4, unsigned(ix0));
        }
        __syncthreads();

        // per-thread loader coordinates: pixel slots and their geometry
        long long pbase[PIX_SLOTS];
        int piy[PIX_SLOTS], pix[PIX_SLOTS];
#pragma unroll
        for (int s = 0; s < PIX_SLOTS; ++s) {
            const int p = (s * kWarps + warp) * 4 + p_lo;
            unsigned ty, tx;
            asm volatile("ld.shared.u64 %0, [%1];" : "=l"(pbase[s]) : "r"(sPixBase + p * 8));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(ty) : "r"(sPixY + p * 4));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tx) : "r"(sPixX + p * 4));
            piy[s] = int(ty);
            pix[s] = int(tx);
        }

        int acc[kPixPerLane];         // REF: the bits of the fp32 running total
#pragma unroll
        for (int i = 0; i < kPixPerLane; ++i) acc[i] = 0;

        const int n_chunks = (P.K + kKC - 1) / kKC;
        const int kq_total = (P.K + 3) / 4;
        float4 a_stage[A_ITERS];   // raw fp32 taps of the next chunk, quantised when stored
        uint4 w_stage[W_ITERS];

        // Issue the global loads of chunk `ch` (activation taps and filter-program quads).
        auto load_chunk = [&](int ch) {
            const int k0 = ch * kKC;
#pragma unroll
            for (int h = 0; h < kLQ / 8; ++h) {
                const int l0 = k0 + (h * 8 + lq_lo) * 4;
                if (P.vec_ok) {
                    const int tap = l0 / P.C;
                    const int c = l0 - tap * P.C;
                    const int ky = tap / P.KW;
                    const int kx = tap - ky * P.KW;
                    const int dy = ky * P.dh, dx = kx * P.dw;
                    const long long toff = ((long long)dy * P.W + dx) * P.C + c;
#pragma unroll
                    for (int s = 0; s < PIX_SLOTS; ++s) {
                        const int iy = piy[s] + dy, ix = pix[s] + dx;
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (l0 < P.K && iy >= 0 && iy < P.H && ix >= 0 && ix < P.W &&
                            AXC_GLOBAL_OK(pbase[s] + toff + 3, (long long)P.N * P.H * P.W * P.C, 211u))
                            v = __ldg(reinterpret_cast<const float4 *>(P.input + pbase[s] + toff));
                        v.x = max_keep_nan(v.x, P.in_floor); v.y = max_keep_nan(v.y, P.in_floor);
                        v.z = max_keep_nan(v.z, P.in_floor); v.w = max_keep_nan(v.w, P.in_floor);
                        a_stage[h * PIX_SLOTS + s] = v;
                    }
                } else {
                    float vals[PIX_SLOTS][4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int l = l0 + e;
                        const int tap = l / P.C;
                        const int c = l - tap * P.C;
                        const int ky = tap / P.KW;
                        const int kx = tap - ky * P.KW;
                        const int dy = ky * P.dh, dx = kx * P.dw;
                        const long long toff = ((long long)dy * P.W + dx) * P.C + c;
#pragma unroll
                        for (int s = 0; s < PIX_SLOTS; ++s) {
                            const int iy = piy[s] + dy, ix = pix[s] + dx;
                            float v = 0.f;
                            if (l < P.K && iy >= 0 && iy < P.H && ix >= 0 && ix < P.W &&
                                AXC_GLOBAL_OK(pbase[s] + toff, (long long)P.N * P.H * P.W * P.C, 212u))
                                v = __ldg(P.input + pbase[s] + toff);
                            vals[s][e] = max_keep_nan(v, P.in_floor);
                        }
                    }
#pragma unroll
                    for (int s = 0; s < PIX_SLOTS; ++s)
                        a_stage[h * PIX_SLOTS + s] = make_float4(vals[s][0], vals[s][1], vals[s][2], vals[s][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < W_ITERS; ++i) {
                const int e = i * kThreads + tid;
                const int lq = e / TN, jj = e - lq * TN;
                const int lqg = ch * kLQ + lq, j = j0 + jj;
                uint4 v;
                if (lqg >= kq_total) v = make_uint4(kProgPadK, kProgPadK, kProgPadK, kProgPadK);
                else if (j >= P.Cout) v = make_uint4(kProgPadN, kProgPadN, kProgPadN, kProgPadN);
                else v = __ldg(P.prog + (size_t)lqg * P.Cout + j);
                w_stage[i] = v;
            }
        };

        // Quantise the staged taps of chunk `ch` and publish the tiles.
        // A tap with l >= K stores byte 0: with the K-tail program word it addresses the zero word.
        auto store_chunk = [&](int ch, int buf) {
            const int k0 = ch * kKC;
#pragma unroll
            for (int h = 0; h < kLQ / 8; ++h)
#pragma unroll
                for (int s = 0; s < PIX_SLOTS; ++s) {
                    const int lq = h * 8 + lq_lo;
                    const int l0 = k0 + lq * 4;
                    const int p = (s * kWarps + warp) * 4 + p_lo;
                    const float4 v = a_stage[h * PIX_SLOTS + s];
                    uint32_t packed = 0;
                    if (l0 + 0 < P.K) packed |= quantize_u8(v.x, Q.in_off, Q.in_inv);
                    if (l0 + 1 < P.K) packed |= quantize_u8(v.y, Q.in_off, Q.in_inv) << 8;
                    if (l0 + 2 < P.K) packed |= quantize_u8(v.z, Q.in_off, Q.in_inv) << 16;
                    if (l0 + 3 < P.K) packed |= quantize_u8(v.w, Q.in_off, Q.in_inv) << 24;
                    sts_u32(sA + buf * A_BYTES + (lq * AROW + p) * 4, packed);
                }
#pragma unroll
            for (int i = 0; i < W_ITERS; ++i) {
                const int e = i * kThreads + tid;
                sts_v4(sW + buf * W_BYTES + e * 16, w_stage[i]);
            }
        };

        // Patch sums (the reference's outCoeffs, tf2/src/approx_nn_conv_kernels.cpp:294): one thread per
        // pixel adds the raw taps of chunk `ch` in l order, so the fp32 sum has the reference's rounding.
        // The running value lives in shared memory; successive chunks are taken by different warps.
        auto patch_sum_chunk = [&](int ch) {
            const int p = (warp % SUM_WARPS) * 32 + lane;
            long long base;
            unsigned ty, tx;
            asm volatile("ld.shared.u64 %0, [%1];" : "=l"(base) : "r"(sPixBase + p * 8));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(ty) : "r"(sPixY + p * 4));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tx) : "r"(sPixX + p * 4));
            const int iy0 = int(ty), ix0 = int(tx);
            float sum = ch == 0 ? 0.0f : lds_f32(sAsum + p * 4);
            const int l_begin = ch * kKC;
            const int l_end = min(P.K, l_begin + kKC);
            int tap = l_begin / P.C;
            int c = l_begin - tap * P.C;
            int ky = tap / P.KW;
            int kx = tap - ky * P.KW;
            if (P.vec_ok) {
                for (int l = l_begin; l < l_end; l += 16) {
                    float4 v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[e] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (l + 4 * e < l_end) {
                            const int iy = iy0 + ky * P.dh, ix = ix0 + kx * P.dw;
                            if (iy >= 0 && iy < P.H && ix >= 0 && ix < P.W)
                                v[e] = __ldg(reinterpret_cast<const float4 *>(
                                    P.input + base + ((long long)(ky * P.dh) * P.W + kx * P.dw) * P.C + c));
                            c += 4;
                            if (c >= P.C) { c = 0; if (++kx >= P.KW) { kx = 0; ++ky; } }
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sum = __fadd_rn(sum, max_keep_nan(v[e].x, P.in_floor));
                        sum = __fadd_rn(sum, max_keep_nan(v[e].y, P.in_floor));
                        sum = __fadd_rn(sum, max_keep_nan(v[e].z, P.in_floor));
                        sum = __fadd_rn(sum, max_keep_nan(v[e].w, P.in_floor));
                    }
                }
            } else {
                for (int l = l_begin; l < l_end; l += 4) {
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[e] = 0.f;
                        if (l + e < l_end) {
                            const int iy = iy0 + ky * P.dh, ix = ix0 + kx * P.dw;
                            if (iy >= 0 && iy < P.H && ix >= 0 && ix < P.W)
                                v[e] = __ldg(P.input + base + ((long long)(ky * P.dh) * P.W + kx * P.dw) * P.C + c);
                            if (++c >= P.C) { c = 0; if (++kx >= P.KW) { kx = 0; ++ky; } }
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) sum = __fadd_rn(sum, max_keep_nan(v[e], P.in_floor));
                }
            }
            sts_f32(sAsum + p * 4, sum);
        };

        load_chunk(0);
        store_chunk(0, 0);
        __syncthreads();

        for (int ch = 0; ch < n_chunks; ++ch) {
            const int buf = ch & 1;
            const bool more = ch + 1 < n_chunks;
            if (more) load_chunk(ch + 1);
            if (warp / SUM_WARPS == ch % SUM_GROUPS) patch_sum_chunk(ch);

            const unsigned aBase = sA + buf * A_BYTES + wm * kPixPerLane * 4;
            const unsigned wBase = sW + buf * W_BYTES + (wn * 32 + lane) * 16;
#pragma unroll 2
            for (int lq = 0; lq < kLQ; ++lq) {
                const uint4 wv = lds_v4(wBase + lq * TN * 16);
#pragma unroll
                for (int pg = 0; pg < kPixPerLane / 4; ++pg) {
                    const uint4 av = lds_v4(aBase + (lq * AROW + pg * 4) * 4);
                    const unsigned aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int pp = 0; pp < 4; ++pp) {
                        if (REF) {
                            float s = __int_as_float(acc[pg * 4 + pp]);
                            s = __fadd_rn(s, entry_to_float(lds_u16(__byte_perm(wv.x, aw[pp], 0x3240))));
                            s = __fadd_rn(s, entry_to_float(lds_u16(__byte_perm(wv.y, aw[pp], 0x3250))));
                            s = __fadd_rn(s, entry_to_float(lds_u16(__byte_perm(wv.z, aw[pp], 0x3260))));
                            s = __fadd_rn(s, entry_to_float(lds_u16(__byte_perm(wv.w, aw[pp], 0x3270))));
                            acc[pg * 4 + pp] = __float_as_int(s);
                        } else {
                            int s = acc[pg * 4 + pp];
                            s += int(lds_u16(__byte_perm(wv.x, aw[pp], 0x3240)));
                            s += int(lds_u16(__byte_perm(wv.y, aw[pp], 0x3250)));
                            s += int(lds_u16(__byte_perm(wv.z, aw[pp], 0x3260)));
                            s += int(lds_u16(__byte_perm(wv.w, aw[pp], 0x3270)));
                            acc[pg * 4 + pp] = s;
                        }
                    }
                }
            }

            if (more) store_chunk(ch + 1, buf ^ 1);
            __syncthreads();
        }

        // ---- dequantisation: ((S*s1s2 + m2*aSum) + m1*bSum) - K*m1m2 -----------------
        const int j = j0 + wn * 32 + lane;
        if (j < P.Cout) {
            const float t2 = __fmul_rn(Q.m1, __ldg(P.bsum + j));
#pragma unroll
            for (int i = 0; i < kPixPerLane; ++i) {
                const long long p = m0 + wm * kPixPerLane + i;
                if (p < P.M && AXC_GLOBAL_OK(p * P.Cout + j, P.M * P.Cout, 213u)) {
                    const float a_sum = lds_f32(sAsum + (wm * kPixPerLane + i) * 4);
                    const float total = REF ? __int_as_float(acc[i]) : float(acc[i]);
                    const float t0 = __fmul_rn(total, Q.s1s2);
                    const float t1 = __fmul_rn(Q.m2, a_sum);
                    P.output[p * P.Cout + j] = __fsub_rn(__fadd_rn(__fadd_rn(t0, t1), t2), Q.km1m2);
                    asm volatile("" ::: "memory");      // the tap may be the same memory (integer sums only): keep the order
                    if (P.acc_out) P.acc_out[p * P.Cout + j] = REF ? __float2int_rz(total) : acc[i];
                }
            }
        }
    }
}

// What the op's callers add to its output, in one pass after the convolution: out = out (+ bias[channel])
// (+ residual), then the ReLU if asked for.  It is a pass of its own because inside the lookup kernels even two more
// instructions per output cost more than this pass (measured on the ResNet-50-shaped network: +1.3 % kernel time
// for a bias add and a max; a shortcut load in the epilogue took a 1x1 layer with 64 input channels from 2.75 to 5.0 ms).
__global__ void __launch_bounds__(256) post_kernel(float *__restrict__ out, const float *__restrict__ bias, const float *__restrict__ residual,
                                                   long long count, int channels, int relu)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(bias)) & 15u) == 0 &&
                     channels % 4 == 0;
    const long long quads = vec ? count / 4 : 0;
    const float floor = relu ? 0.0f : -INFINITY;
    for (long long q = tid; q < quads; q += nthreads) {
        float4 a = reinterpret_cast<const float4 *>(out)[q];
        if (bias) {
            const float4 b = __ldg(reinterpret_cast<const float4 *>(bias) + (q % (channels / 4)));
            a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
        }
        if (residual) {
            const float4 b = __ldg(reinterpret_cast<const float4 *>(residual) + q);
            a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
        }
        a.x = max_keep_nan(a.x, floor); a.y = max_keep_nan(a.y, floor); a.z = max_keep_nan(a.z, floor); a.w = max_keep_nan(a.w, floor);
        reinterpret_cast<float4 *>(out)[q] = a;
    }
    for (long long e = quads * 4 + tid; e < count; e += nthreads) {
        float y = out[e];
        if (bias) y = __fadd_rn(y, __ldg(bias + e % channels));
        if (residual) y = __fadd_rn(y, __ldg(residual + e));
        out[e] = max_keep_nan(y, floor);
    }
}

template <int WN, bool REF>
int launch_dense_variant(const DenseParams &P, const DeviceInfo &di, cudaStream_t stream)
{
    constexpr int TM = (kWarps / WN) * kPixPerLane;
    constexpr int TN = WN * 32;
    DenseParams Q = P;
    Q.tiles_n = (P.Cout + TN - 1) / TN;
    Q.tiles_total = ((P.M + TM - 1) / TM) * Q.tiles_n;
    AXC_CUDA(cudaFuncSetAttribute(dense_kernel<WN, REF>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
    const long long grid = Q.tiles_total < di.sm_count ? Q.tiles_total : di.sm_count;
    dense_kernel<WN, REF><<<unsigned(grid), kThreads, size_t(di.max_smem_optin), stream>>>(Q);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    return AXC_OK;
}

}  // namespace

int launch_post(float *out, const float *bias, const float *residual, long long count, int channels, int relu,
                const DeviceInfo &di, cudaStream_t stream)
{
    if (count <= 0) return AXC_OK;
    const long long want = (count / 4 + 255) / 256;
    const unsigned blocks = unsigned(want < (long long)di.sm_count * 8 ? (want > 0 ? want : 1) : (long long)di.sm_count * 8);
    post_kernel<<<blocks, 256, 0, stream>>>(out, bias, residual, count, channels > 0 ? channels : 1, relu);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    return AXC_OK;
}

// 0 = bank-scheduled kernel with the common-K kernel as its device-side fallback (default),
// 1 = common-K kernel only.  Read once from AXC_DENSE_VARIANT.
AXC_DEFINE_BOUNDS_READER(bounds_record_conv)

static int dense_variant()
{
    static const int v = [] {
        const char *e = getenv("AXC_DENSE_VARIANT");
        return (e && e[0] == '1') ? 1 : 0;
    }();
    return v;
}

int launch_dense(const uint16_t *lut_dev, unsigned table_uid, const Geom &g, const Quant &q, const float *ranges_dev,
                 const float *input, const float *filter, float *output, void *workspace, const axc_debug_out *dbg,
                 int device, cudaStream_t stream, bool ref_order)
{
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    // A caller that wants the integer sums only (output == NULL, the quantised entry point) gets the fp32 value written
    // to the same element of the accumulator tap first and the integer sum over it: the kernels need no test per store.
    const bool ints_only = output == nullptr;
    if (ints_only) {
        if (!dbg || !dbg->acc) return AXC_INVALID_ARGUMENT;
        output = reinterpret_cast<float *>(dbg->acc);
    }
    // The kernels are laid out for the 227 KiB of sm_100 and address the table by absolute window addresses: refuse
    // to launch where the probed window of this device does not start early enough or does not reach 228 KiB
    // (a kernel that found its layout broken would leave the output unwritten).
    if (di.max_smem_optin < 232448 || di.smem_base > 2048u || di.smem_end < 233472u) return AXC_INTERNAL;
    // the scheduled kernel divides by C and KW with 40-bit reciprocals, exact while K * max(C, KW) < 2^40; it
    // lets every lane walk K in an order of its own, so a sum that has to be taken in K order is not its job
    const bool scheduled = !ref_order && g.plan == AXC_PLAN_KEEP && dense_variant() == 0 && (long long)g.K * (g.C > g.KW ? g.C : g.KW) < (1ll << 40);
    const PlanLayout L = plan_layout(g.K, g.Cout);
    const Workspace ws = dense_workspace(g.K, g.Cout);
    unsigned char *plan = static_cast<unsigned char *>(workspace);
    unsigned char *wsb = plan + L.total;
    uint4 *prog = reinterpret_cast<uint4 *>(wsb);
    float *bsum = reinterpret_cast<float *>(wsb + ws.sums_off);
    int *status = reinterpret_cast<int *>(wsb + ws.status_off);
    const int *gate = nullptr;
    const DevQuant *dq = reinterpret_cast<const DevQuant *>(plan + kDevQuantOffset);

    // the quantisation parameters reach the workspace with the first kernel of the plan check, or - without a
    // plan - with a kernel of their own
    if (scheduled) rc = launch_plan(lut_dev, table_uid, g, q, ranges_dev, filter, plan, L, dbg ? dbg->qfilter : nullptr, stream);
    else rc = launch_quant(q, ranges_dev, g.K, plan, stream);
    if (rc) return rc;
    if (dbg && dbg->qinput) {
        const long long n = (long long)g.N * g.H * g.W * g.C;
        if (n > 0) {
            const unsigned blocks = unsigned(n / 256 + 1 < 4096 ? n / 256 + 1 : 4096);
            quantize_tensor_kernel<<<blocks, 256, 0, stream>>>(input, n, dq, dbg->qinput, g.ep.input_relu ? 0.0f : -INFINITY);
            AXC_CUDA(cudaGetLastError());
            count_launch();
        }
    }
    if (scheduled) {
        rc = launch_dense_sched(g, input, output, plan, L, dbg ? dbg->acc : nullptr, di, stream);
        if (rc) return rc;
        gate = &reinterpret_cast<const PlanHeader *>(plan)->fallback;
    }
    {
        const long long items = (long long)((g.K + 3) / 4) * g.Cout;
        const unsigned blocks = unsigned((items + 255) / 256);
        filter_prep_kernel<<<blocks, 256, 0, stream>>>(filter, g.K, g.Cout, dq, prog,
                                                       (dbg && !scheduled) ? dbg->qfilter : nullptr, status, gate);
        AXC_CUDA(cudaGetLastError());
        filter_sum_kernel<<<unsigned((g.Cout + 31) / 32), 32, 0, stream>>>(filter, g.K, g.Cout, bsum, gate);
        AXC_CUDA(cudaGetLastError());
        count_launch(2);
    }

    DenseParams P;
    P.lut = lut_dev; P.input = input; P.output = output; P.prog = prog; P.bsum = bsum;
    P.acc_out = dbg ? dbg->acc : nullptr;
    P.status = status;
    P.gate = gate;
    P.in_floor = g.ep.input_relu ? 0.0f : -INFINITY;
    P.N = g.N; P.H = g.H; P.W = g.W; P.C = g.C; P.KH = g.KH; P.KW = g.KW; P.Cout = g.Cout;
    P.sh = g.sh; P.sw = g.sw; P.dh = g.dh; P.dw = g.dw; P.ph = g.ph; P.pw = g.pw; P.OH = g.OH; P.OW = g.OW;
    P.K = g.K; P.M = g.M;
    P.tiles_n = 0; P.tiles_total = 0;
    P.dq = dq;
    P.vec_ok = (g.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(input) & 15u) == 0);
    if (ref_order) rc = g.Cout <= 32 ? launch_dense_variant<1, true>(P, di, stream) : launch_dense_variant<2, true>(P, di, stream);
    else rc = g.Cout <= 32 ? launch_dense_variant<1, false>(P, di, stream) : launch_dense_variant<2, false>(P, di, stream);
    if (rc == AXC_OK && !ints_only && (g.ep.bias || g.ep.residual || g.ep.relu))
        rc = launch_post(output, g.ep.bias, g.ep.residual, g.M * g.Cout, g.Cout, g.ep.relu, di, stream);
    return rc;
}

}  // namespace axc

extern "C" int axc_add_residual(float *out, const float *residual, size_t count, int relu, int device, void *stream)
{
    using namespace axc;
    if (count > 0 && (!out || !residual)) return AXC_INVALID_ARGUMENT;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    rc = launch_post(out, nullptr, residual, (long long)count, 1, relu, di, cudaStream_t(stream));
    if (prev != device) cudaSetDevice(prev);
    return rc;
}
