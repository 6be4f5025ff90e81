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
#include <cuda.h>

#include <cmath>

#include <mutex>
#include <type_traits>

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
    const uint32_t *prog_packed;  // [(KH*KW+1)/2][OC]: bytes {column, plane} of tap 2i, then of tap 2i+1
    const float *bsum;     // [OC]
    int32_t *acc_out;
    int *status;
    int N, H, W, C, KH, KW, mult, OC;
    int sh, sw, dh, dw, ph, pw, OH, OW;
    int run;               // output pixels per warp item
    int runs_per_row, groups;
    long long items;       // N*OH*runs_per_row*groups
    float in_off, in_inv, s1s2, m1, m2, km1m2;
    // expanded-table kernel only
    const float *filter;   // [9][OC] fp32
    float f_off, f_inv;
    int bands;             // bands of output rows per image
    int units_per_group;   // N * bands
    int wave, sets;        // CTAs per set (= channel groups served at a time) and sets: grid = wave * sets
    Epilogue ep;           // fused additions to the output
    float in_floor;        // every input element is max(x, in_floor) as it is loaded: 0 = the producer's ReLU, -inf = none
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
                                      uint32_t *__restrict__ prog, uint32_t *__restrict__ prog_packed,
                                      float *__restrict__ bsum, uint8_t *__restrict__ qfilter, int *status)
{
    const int oc = blockIdx.x * blockDim.x + threadIdx.x;
    if (oc == 0) *status = 0;
    if (oc >= OC) return;
    float s = 0.0f;
    unsigned packed = 0;
    for (int t = 0; t < KHW; ++t) {
        const float f = filter[(size_t)t * OC + oc];
        s = __fadd_rn(s, f);
        const unsigned b = dw_quantize_u8(f, f_off, f_inv);
        prog[(size_t)t * OC + oc] = ((b & 127u) << 1) | ((1u + (b >> 7)) << 16);
        const unsigned half = ((b & 127u) << 1) | ((1u + (b >> 7)) << 8);
        packed = (t & 1) ? (packed | (half << 16)) : half;
        if ((t & 1) || t == KHW - 1) prog_packed[(size_t)(t >> 1) * OC + oc] = (t & 1) ? packed : (packed | (1u << 24));
        if (qfilter) qfilter[(size_t)t * OC + oc] = uint8_t(b);
    }
    bsum[oc] = s;
}

__global__ void dw_quantize_tensor_kernel(const float *__restrict__ x, long long n, float off, float inv,
                                          uint8_t *__restrict__ q, float in_floor)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) q[i] = uint8_t(dw_quantize_u8(max_keep_nan(x[i], in_floor), off, inv));
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

__device__ __forceinline__ float dw_epilogue(int acc, float a_sum, float t2, const DwParams &P, int oc, long long idx)
{
    const float t0 = __fmul_rn(float(acc), P.s1s2);
    const float t1 = __fmul_rn(P.m2, a_sum);
    const float y = __fsub_rn(__fadd_rn(__fadd_rn(t0, t1), t2), P.km1m2);
    return apply_epilogue(y, P.ep, P.ep.bias ? __ldg(P.ep.bias + oc) : 0.0f, idx);
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
                    v = max_keep_nan(__ldg(P.input + (((long long)n * P.H + iy) * P.W + ix) * P.C + c), P.in_floor);
                a_sum = __fadd_rn(a_sum, v);
                const unsigned qa = dw_quantize_u8(v, P.in_off, P.in_inv);
                const unsigned w = __ldg(P.prog + (size_t)tap * P.OC + oc);
                acc += int(dw_lds_u16(__byte_perm(w, qa, 0x3240)));
            }
            const long long o = (((long long)n * P.OH + oh) * P.OW + ow) * P.OC + oc;
            P.output[o] = dw_epilogue(acc, a_sum, t2, P, oc, o);
            if (P.acc_out) P.acc_out[o] = acc;
        }
    }
}

// prmt.b32 with an immediate selector (a selector nibble with bit 3 set replicates the sign of the byte)
template <unsigned SEL>
__device__ __forceinline__ unsigned dw_prmt(unsigned a, unsigned b)
{
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "n"(SEL));
    return d;
}

// Table address of tap TAP (0..8) for the activation in byte SLOT of `q`.  `wp` packs the program bytes of two
// taps: {column byte, plane byte} of tap 2i in bytes 0-1 and of tap 2i+1 in bytes 2-3.  Result bytes:
// {column, activation, plane, 0}; the zero is the replicated sign bit of the plane byte (1 or 2).
template <int TAP, int SLOT>
__device__ __forceinline__ unsigned dw_addr(const unsigned *wp, unsigned q)
{
    constexpr unsigned lo = (TAP & 1) ? 2u : 0u;                 // column byte of this tap inside wp[TAP/2]
    constexpr unsigned sel = lo | ((4u + SLOT) << 4) | ((lo + 1u) << 8) | ((8u | (lo + 1u)) << 12);
    return dw_prmt<sel>(wp[TAP >> 1], q);
}

// Nine table MACs and the raw-tap sum of one output, taps in (ky, kx) order; U = position of the output in
// its batch of three, which fixes the ring slot of every logical column at compile time.
template <int S, int U>
__device__ __forceinline__ float dw_window(const float (&xf)[3][3], const unsigned (&xq)[3], const unsigned *wp, int *acc_out)
{
    constexpr int c0 = (S * U + 0) % 3, c1 = (S * U + 1) % 3, c2 = (S * U + 2) % 3;
    float a = 0.0f;
    int acc = 0;
    a = __fadd_rn(a, xf[0][c0]); acc += int(dw_lds_u16(dw_addr<0, c0>(wp, xq[0])));
    a = __fadd_rn(a, xf[0][c1]); acc += int(dw_lds_u16(dw_addr<1, c1>(wp, xq[0])));
    a = __fadd_rn(a, xf[0][c2]); acc += int(dw_lds_u16(dw_addr<2, c2>(wp, xq[0])));
    a = __fadd_rn(a, xf[1][c0]); acc += int(dw_lds_u16(dw_addr<3, c0>(wp, xq[1])));
    a = __fadd_rn(a, xf[1][c1]); acc += int(dw_lds_u16(dw_addr<4, c1>(wp, xq[1])));
    a = __fadd_rn(a, xf[1][c2]); acc += int(dw_lds_u16(dw_addr<5, c2>(wp, xq[1])));
    a = __fadd_rn(a, xf[2][c0]); acc += int(dw_lds_u16(dw_addr<6, c0>(wp, xq[2])));
    a = __fadd_rn(a, xf[2][c1]); acc += int(dw_lds_u16(dw_addr<7, c1>(wp, xq[2])));
    a = __fadd_rn(a, xf[2][c2]); acc += int(dw_lds_u16(dw_addr<8, c2>(wp, xq[2])));
    *acc_out = acc;
    return a;
}

// 3x3, dilation 1, stride S in {1, 2}.  Lane = output channel; a warp walks a run of output pixels of one row.
// The 3x3 window lives in registers: raw fp32 taps in three ring slots per filter row (output u of a batch of
// three reads logical column kx from slot (S*u + kx) % 3, so sliding costs no moves) and the quantised taps
// packed as one byte per slot in one register per filter row.  The new columns of a whole batch are requested
// before its first output is computed.  Offsets are 32-bit: the launcher sends tensors of 2^31 elements or more
// to the generic kernel.
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
    const int items = int(P.items);
    for (int item = blockIdx.x * kDwWarps + warp; item < items; item += gridDim.x * kDwWarps) {
        const int grp = item % P.groups;
        int t = item / P.groups;
        const int r = t % P.runs_per_row;
        t /= P.runs_per_row;
        const int oh = t % P.OH;
        const int n = t / P.OH;
        const int oc = grp * 32 + lane;
        if (oc >= P.OC) continue;
        const int c = oc / P.mult;
        const float t2 = __fmul_rn(P.m1, __ldg(P.bsum + oc));
        unsigned wp[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) wp[i] = __ldg(P.prog_packed + i * P.OC + oc);

        const int ow0 = r * P.run;
        const int ow_end = min(P.OW, ow0 + P.run);
        const int iy0 = oh * P.sh - P.ph;
        const int ix_first = ow0 * S - P.pw;              // leftmost input column of the first window
        int rowoff[3];                                    // element offset of (row, column ix_first, channel c)
        bool rowok[3];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const int iy = iy0 + ky;
            rowok[ky] = unsigned(iy) < unsigned(P.H);
            rowoff[ky] = (((n * P.H + (rowok[ky] ? iy : 0)) * P.W) + ix_first) * P.C + c;
        }
        int outoff = ((n * P.OH + oh) * P.OW + ow0) * P.OC + oc;

        float xf[3][3];       // [ky][slot]
        unsigned xq[3] = {0u, 0u, 0u};   // [ky], byte = slot
        // columns 0 .. 2-S of the first window
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
            for (int kx = 0; kx < 3 - S; ++kx) {
                const bool ok = rowok[ky] && unsigned(ix_first + kx) < unsigned(P.W);
                xf[ky][kx] = ok ? max_keep_nan(__ldg(P.input + (rowoff[ky] + kx * P.C)), P.in_floor) : 0.0f;
                xq[ky] |= dw_quantize_u8(xf[ky][kx], P.in_off, P.in_inv) << (8 * kx);
            }
        int col = 3 - S;                                  // next new column, relative to ix_first
        for (int owb = ow0; owb < ow_end; owb += 3) {
            float nf[3][S][3];                            // [output of the batch][new column][ky]
#pragma unroll
            for (int u = 0; u < 3; ++u)
#pragma unroll
                for (int k2 = 0; k2 < S; ++k2) {
                    const int rel = col + u * S + k2;
                    const bool colok = owb + u < ow_end && unsigned(ix_first + rel) < unsigned(P.W);
                    const int o = rel * P.C;
#pragma unroll
                    for (int ky = 0; ky < 3; ++ky)
                        nf[u][k2][ky] = (colok && rowok[ky]) ? max_keep_nan(__ldg(P.input + (rowoff[ky] + o)), P.in_floor) : 0.0f;
                }
            col += 3 * S;
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                if (owb + u < ow_end) {
#pragma unroll
                    for (int k2 = 0; k2 < S; ++k2) {
                        const int slot = (S * u + (3 - S) + k2) % 3;
#pragma unroll
                        for (int ky = 0; ky < 3; ++ky) {
                            xf[ky][slot] = nf[u][k2][ky];
                            const unsigned q = dw_quantize_u8(nf[u][k2][ky], P.in_off, P.in_inv);
                            xq[ky] = (xq[ky] & ~(0xFFu << (8 * slot))) | (q << (8 * slot));
                        }
                    }
                    // taps in the reference's order (ky, kx); logical column kx sits in slot (S*u + kx) % 3
                    float a_sum = 0.0f;
                    int acc = 0;
                    if (u == 0) {
                        a_sum = dw_window<S, 0>(xf, xq, wp, &acc);
                    } else if (u == 1) {
                        a_sum = dw_window<S, 1>(xf, xq, wp, &acc);
                    } else {
                        a_sum = dw_window<S, 2>(xf, xq, wp, &acc);
                    }
                    P.output[outoff] = dw_epilogue(acc, a_sum, t2, P, oc, outoff);
                    if (P.acc_out) P.acc_out[outoff] = acc;
                    outoff += P.OC;
                }
            }
        }
    }
}


// ---------------------------------------------------------------------------------------------------
// 3x3 depthwise with a per-channel-group expanded table (stride 1 or 2, dilation 1).
//
// In the kernels above activation and weight both differ from lane to lane, so the bank of a lookup is random
// (3.2 wavefronts per lookup measured).  A depthwise lane, however, only ever uses the nine table columns of its
// own channel.  For a group of 32 channels the CTA therefore expands the table once into
//     T16[a][lane] = the entries LUT[a][b(lane, tap)] of eight taps, 16 bytes,   T4[a][lane] = the centre tap,
// (160 KiB of shared memory) and then looks an INPUT pixel up instead of an output tap: one LDS.128 plus one
// LDS.32 return all nine products of the pixel, which are scattered to the nine outputs it contributes to.  The
// address is a * 512 + lane * 16: the bank depends on the lane alone, so every quarter warp of the LDS.128 and the
// whole LDS.32 are conflict-free - 5 wavefronts per 9 table MACs instead of 29.
//
// Work: the CTA owns a contiguous range of (channel group, image, band of R output rows) units; it rebuilds the
// table when the range crosses into the next group.  A warp walks a band from left to right, lane = channel: per
// input column it loads the (R-1)*S+3 rows of the column (one 128-byte line each), quantises, looks up and adds
// the products into the accumulators of the (at most) three output columns in flight; a finished output column
// gets its patch sum - the raw taps added in (ky, kx) order like the reference's im2col
// (tf2/src/approx_nn_conv_kernels.cpp:272-295) - and is dequantised and stored.
//
// Packing of a T16 entry: x = {t00, t02}, y = {t20, t22}, z = {t01, t21}, w = {t10, t12} (low half first), so
// that under stride 2 a pixel fetches only what its row and column parity can use (8, 4, 4 or 4 bytes).
// ---------------------------------------------------------------------------------------------------
constexpr unsigned kTab16Bytes = 256u * 32u * 16u;
constexpr unsigned kTab4Bytes = 256u * 32u * 4u;
constexpr unsigned kTabSmem = kTab16Bytes + kTab4Bytes + 512u;
constexpr int kPlainL2Ahead = 3;   // the same for the kernel that fetches with plain loads
constexpr int kTmaL2Ahead = 6;     // columns ahead of the copy in flight that are prefetched into L2
constexpr long long kTabMinOutputsPerGroup = 32768;

__device__ __forceinline__ unsigned dw_q_u8(float x, float off, float inv)
{
    const float v = __fadd_rn(__fmul_rn(__fsub_rn(x, off), inv), 0.5f);
    unsigned u;
    asm("cvt.rzi.u8.f32 %0, %1;" : "=r"(u) : "f"(v));     // truncates and saturates to 0..255 (NaN -> 0)
    return u;
}

// c + low / high 16-bit half of `a`: one two-way dot product with the byte vector {1,0} resp. {0,1} (measured no
// slower than mask / shift + add, and one instruction instead of two)
__device__ __forceinline__ int dw_add_lo(unsigned a, int c)
{
    int d;
    asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(0x00000001u), "r"(c));
    return d;
}
__device__ __forceinline__ int dw_add_hi(unsigned a, int c)
{
    int d;
    asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(0x00000100u), "r"(c));
    return d;
}

template <int NT>
__device__ __forceinline__ void dw_build_table(const DwParams &P, int g, unsigned tab16, unsigned tab4, int tid)
{
    constexpr int kTabWarps = NT / 32;
    const int lane = tid & 31;
    const int oc = g * 32 + lane;
    unsigned b[9];
#pragma unroll
    for (int t = 0; t < 9; ++t) b[t] = oc < P.OC ? dw_q_u8(__ldg(P.filter + (size_t)t * P.OC + oc), P.f_off, P.f_inv) : 0u;
#pragma unroll 4
    for (int a = tid >> 5; a < 256; a += kTabWarps) {
        const uint16_t *row = P.lut + a * 256;
        unsigned t[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) t[k] = __ldg(row + b[k]);
        const unsigned d16 = tab16 + unsigned(a) * 512u + unsigned(lane) * 16u;
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(d16), "r"(t[0] | (t[2] << 16)), "r"(t[6] | (t[8] << 16)),
                     "r"(t[1] | (t[7] << 16)), "r"(t[3] | (t[5] << 16)) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(tab4 + unsigned(a) * 128u + unsigned(lane) * 4u), "r"(t[4]) : "memory");
    }
}

// base + a * b for an unsigned 32-bit a * b and a 64-bit base: one instruction (IMAD.WIDE)
__device__ __forceinline__ const char *dw_ptr_mad(const char *base, unsigned a, unsigned b)
{
    unsigned long long r;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"(a), "r"(b), "l"((unsigned long long)base));
    return reinterpret_cast<const char *>(r);
}

// ---- TMA helpers: every column of a band (IR rows x 32 channels) is one tiled bulk copy into a stage buffer of the
// warp; rows, columns and channels outside the tensor arrive as zeros, which is exactly the padding rule ----------
__device__ __forceinline__ void dw_mbar_init(unsigned bar)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void dw_tma_column(unsigned dst, const CUtensorMap *tmap, unsigned bar, unsigned bytes, int x, int col, int row, int n)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(col), "r"(row), "r"(n), "r"(bar) : "memory");
}
__device__ __forceinline__ void dw_tma_prefetch_l2(const CUtensorMap *tmap, int x, int col, int row, int n)
{
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap), "r"(x), "r"(col), "r"(row), "r"(n) : "memory");
}
// Waits for the phase `parity` of the barrier, at most about a second; false if the copy never arrived.
__device__ __forceinline__ bool dw_mbar_wait(unsigned bar, unsigned parity)
{
    for (int it = 0; it < (1 << 20); ++it) {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

template <int S, int R, int NT, bool DBG, bool TMA>
__device__ __forceinline__ void depthwise_3x3_tab_body(const DwParams &P, const CUtensorMap *tmap)
{
    constexpr int IR = (R - 1) * S + 3;
    constexpr int kTabWarps = NT / 32;
    constexpr int STAGES = S == 1 ? 3 : 2;          // stage of a column = its index % STAGES: a compile-time slot
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const unsigned dyn0 = (unsigned)__cvta_generic_to_shared(smem_raw);
    unsigned dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    const unsigned tab16 = (dyn0 + 511u) & ~511u;
    const unsigned tab4 = tab16 + kTab16Bytes;
    constexpr unsigned box_bytes = unsigned(IR) * 128u;        // what one copy delivers: IR rows of 32 channels
    constexpr unsigned stage_bytes = box_bytes;                // a multiple of 128 bytes, as the copy's destination must be
    const unsigned stages0 = tab4 + kTab4Bytes;                                        // [warp][stage][row][channel]
    const unsigned bars0 = stages0 + (TMA ? unsigned(kTabWarps * STAGES) * stage_bytes : 0u);   // [warp][stage] mbarriers
    if (bars0 + (TMA ? unsigned(kTabWarps * STAGES) * 8u : 0u) > dyn0 + dyn_size) {
        if (threadIdx.x == 0) atomicExch(P.status, 1);
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned my_stage0 = stages0 + unsigned(warp * STAGES) * stage_bytes;
    const unsigned my_bar0 = bars0 + unsigned(warp * STAGES) * 8u;
    unsigned phase = 0;                 // bit s: parity the next wait on stage s expects
    bool failed = false;                // a copy did not arrive in time: status 3, no further waits
    if (TMA) {
        if (lane == 0) {
#pragma unroll
            for (int st = 0; st < STAGES; ++st) dw_mbar_init(my_bar0 + st * 8u);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
    }
    const unsigned lane16 = tab16 + unsigned(lane) * 16u, lane4 = tab4 + unsigned(lane) * 4u;
    // CTAs work in sets of `wave` = min(groups, CTAs) members: the members of a set take different channel groups of
    // the same range of bands at the same time, so that the 128-byte pieces of a pixel that the groups read lie
    // close together in time as well as in memory.  With more groups than CTAs a member takes several groups in turn.
    const int wave = P.wave, set = int(blockIdx.x) / wave, slot = int(blockIdx.x) - set * wave;
    const int w_begin = int((long long)P.units_per_group * set / P.sets);
    const int w_end = int((long long)P.units_per_group * (set + 1) / P.sets);
    const unsigned row_bytes = unsigned(P.W) * unsigned(P.C) * 4u;        // the launcher keeps IR rows below 2^32 bytes
    const unsigned orow_bytes = unsigned(P.OW) * unsigned(P.OC) * 4u;
    const unsigned pix_bytes = unsigned(P.C) * 4u, opix_bytes = unsigned(P.OC) * 4u;
    const float in_off = P.in_off, in_inv = P.in_inv, s1s2 = P.s1s2, m2 = P.m2, km1m2 = P.km1m2, in_floor = P.in_floor;
    constexpr int PF = kPlainL2Ahead;

    for (int g = slot; g < P.groups; g += wave) {
        __syncthreads();                                    // every warp is done with the previous group's table
        dw_build_table<NT>(P, g, tab16, tab4, tid);
        __syncthreads();

        const int oc = g * 32 + lane;
        const bool oc_ok = oc < P.OC;
        const int cin = oc_ok ? oc / P.mult : 0;
        const float t2 = oc_ok ? __fmul_rn(P.m1, __ldg(P.bsum + oc)) : 0.0f;
        const float bias_j = (oc_ok && P.ep.bias) ? __ldg(P.ep.bias + oc) : 0.0f;

        for (int w = w_begin + warp; w < w_end; w += kTabWarps) {
            const int n = w / P.bands;
            const int oy0 = (w - n * P.bands) * R;
            const int rows_here = oc_ok ? (P.OH - oy0 < R ? P.OH - oy0 : R) : 0;      // rows this lane stores
            const int iy0 = oy0 * S - P.ph;
            // input rows lo <= i < hi of the band lie inside the image (lo is 0 or 1)
            const int lo = iy0 < 0 ? -iy0 : 0;
            const int hi = P.H - iy0 < IR ? P.H - iy0 : IR;
            // byte pointers: input element (n, iy0, image column -pw, cin); output element (n, oy0, 0, oc)
            const char *in0 = reinterpret_cast<const char *>(P.input + ((long long)n * P.H + iy0) * (long long)(P.W * P.C) -
                                                             (long long)P.pw * P.C + cin);
            const long long o0 = ((long long)n * P.OH + oy0) * (long long)(P.OW * P.OC) + (oc_ok ? oc : 0);
            const char *out0 = reinterpret_cast<const char *>(P.output + o0);
            const char *acc0 = DBG ? reinterpret_cast<const char *>(P.acc_out + o0) : nullptr;
            const char *res0 = P.ep.residual ? reinterpret_cast<const char *>(P.ep.residual + o0) : nullptr;

            int acc[R][S == 1 ? 3 : 2];
            float xf[IR][3];      // raw taps of the columns in flight: S == 1 ring slot = column % 3; S == 2: 0 / 1 = even
                                  // columns (m % 2), 2 = odd column
            float nx[IR];         // raw taps of the column being fetched (plain loads only)
            const int ncols = S == 1 ? P.OW + 2 : 2 * P.OW + 1;                   // input columns of the band
            const unsigned lane_off = unsigned(lane) * 4u;

            // TMA: column `c` into stage `st`, issued by lane 0 after the whole warp has consumed the stage
            auto tma_issue = [&](int c, int st) {
                __syncwarp();
                if (lane == 0 && c < ncols) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    dw_tma_column(my_stage0 + unsigned(st) * stage_bytes, tmap, my_bar0 + unsigned(st) * 8u, box_bytes, g * 32,
                                  c - P.pw, iy0, n);
                    if (c + kTmaL2Ahead < ncols) dw_tma_prefetch_l2(tmap, g * 32, c + kTmaL2Ahead - P.pw, iy0, n);
                }
            };
            // TMA: raw taps of the column in stage `st` into xf slot `slot`
            auto tma_take = [&](auto stc, auto slotc) {
                constexpr int st = decltype(stc)::value, slot = decltype(slotc)::value;
                if (!failed) {
                    if (!dw_mbar_wait(my_bar0 + st * 8u, (phase >> st) & 1u)) {
                        failed = true;
                        atomicExch(P.status, 3);
                    }
                    phase ^= 1u << st;
                }
                const unsigned a = my_stage0 + unsigned(st) * stage_bytes + lane_off;
#pragma unroll
                for (int i = 0; i < IR; ++i) {
                    xf[i][slot] = 0.0f;
                    if (AXC_SHARED_OK(a + unsigned(i) * 128u, 4u, stages0, bars0, 307u))
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xf[i][slot]) : "r"(a + unsigned(i) * 128u));
                    if (P.ep.input_relu) xf[i][slot] = fmaxf(xf[i][slot], 0.0f);     // the producer's ReLU (zeros of the padding stay zeros)
                }
            };

            // raw taps of input column `c` (relative: image column c - pw); zeros outside the image
            auto fetch = [&](int c) {
                if (unsigned(c - P.pw) < unsigned(P.W)) {          // the same for all lanes
                    const char *colp = dw_ptr_mad(in0, unsigned(c), pix_bytes);
#pragma unroll
                    for (int i = 0; i < IR; ++i) {
                        float x = 0.0f;
                        if (i >= lo && i < hi) x = max_keep_nan(__ldg(reinterpret_cast<const float *>(dw_ptr_mad(colp, unsigned(i), row_bytes))), in_floor);
                        nx[i] = x;
                    }
                    if (PF > 0 && unsigned(c + PF - P.pw) < unsigned(P.W)) {
                        const char *pfp = colp + PF * pix_bytes;
#pragma unroll
                        for (int i = 0; i < IR; ++i)
                            if (i >= lo && i < hi) asm volatile("prefetch.global.L2 [%0];" ::"l"(dw_ptr_mad(pfp, unsigned(i), row_bytes)));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < IR; ++i) nx[i] = 0.0f;
                }
            };
            // patch sum, dequantisation and store of output column ox, rows 0..R-1: raw columns in xf slots
            // (k0, k1, k2) for kx = 0, 1, 2, integer sums in slot sa
            auto emit = [&](int ox, auto k0c, auto k1c, auto k2c, auto sac) {
                constexpr int k0 = decltype(k0c)::value, k1 = decltype(k1c)::value, k2 = decltype(k2c)::value;
                constexpr int sa = decltype(sac)::value;
                const char *outp = dw_ptr_mad(out0, unsigned(ox), opix_bytes);
                const char *accp = DBG ? dw_ptr_mad(acc0, unsigned(ox), opix_bytes) : nullptr;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    // 0 + x00 of the reference's running sum is x00 up to the sign of a zero, which cannot reach the output
                    float a = xf[r * S][k0];
                    a = __fadd_rn(a, xf[r * S][k1]);
                    a = __fadd_rn(a, xf[r * S][k2]);
#pragma unroll
                    for (int ky = 1; ky < 3; ++ky) {
                        a = __fadd_rn(a, xf[r * S + ky][k0]);
                        a = __fadd_rn(a, xf[r * S + ky][k1]);
                        a = __fadd_rn(a, xf[r * S + ky][k2]);
                    }
                    const float t0 = __fmul_rn(float(acc[r][sa]), s1s2);
                    const float t1 = __fmul_rn(m2, a);
                    float y = __fsub_rn(__fadd_rn(__fadd_rn(t0, t1), t2), km1m2);
                    if (P.ep.bias) y = __fadd_rn(y, bias_j);
                    if (P.ep.residual && r < rows_here)
                        y = __fadd_rn(y, __ldg(reinterpret_cast<const float *>(dw_ptr_mad(dw_ptr_mad(res0, unsigned(ox), opix_bytes), unsigned(r), orow_bytes))));
                    if (P.ep.relu) y = fmaxf(y, 0.0f);
                    // predicated stores (no branch): rows_here is 0 for a lane without a channel
                    if (AXC_GLOBAL_OK(r < rows_here ? o0 + (long long)r * P.OW * P.OC + (long long)ox * P.OC : 0, (long long)P.N * P.OH * P.OW * P.OC, 313u))
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.gt.s32 p, %2, %3;\n\t@p st.global.f32 [%0], %1;\n\t}"
                                 ::"l"(dw_ptr_mad(outp, unsigned(r), orow_bytes)), "f"(y), "r"(rows_here), "r"(r) : "memory");
                    if (DBG)
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.gt.s32 p, %2, %3;\n\t@p st.global.s32 [%0], %1;\n\t}"
                                     ::"l"(dw_ptr_mad(accp, unsigned(r), orow_bytes)), "r"(acc[r][sa]), "r"(rows_here), "r"(r) : "memory");
                }
            };
            using I0 = std::integral_constant<int, 0>;
            using I1 = std::integral_constant<int, 1>;
            using I2 = std::integral_constant<int, 2>;

            if constexpr (S == 1) {
                // Input column c serves kx = 0 of output c, kx = 1 of output c - 1, kx = 2 of output c - 2.  The first
                // product an output receives (ky = 0, kx = 0) initialises its sum, so no slot is ever cleared; what
                // columns 0 and 1 add to the slots of the non-existent outputs -2 and -1 is overwritten that way.
                auto column = [&](int c, auto jc) {
                    constexpr int J = decltype(jc)::value;            // c % 3
                    constexpr int s0 = J, s1 = (J + 2) % 3, s2 = (J + 1) % 3;
                    if (TMA) {
                        tma_take(std::integral_constant<int, J>{}, std::integral_constant<int, J>{});
                    } else {
#pragma unroll
                        for (int i = 0; i < IR; ++i) xf[i][J] = nx[i];
                        fetch(c + 1);                                  // next column in flight while this one is used
                    }
#pragma unroll
                    for (int i = 0; i < IR; ++i) {
                        const unsigned qa = dw_q_u8(xf[i][J], in_off, in_inv);
                        uint4 t = make_uint4(0, 0, 0, 0);
                        if (AXC_SHARED_OK(lane16 + qa * 512u, 16u, tab16, tab16 + kTab16Bytes, 301u))
                            asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.x), "=r"(t.y), "=r"(t.z), "=r"(t.w) : "r"(lane16 + qa * 512u));
                        if (i < R) {                                   // ky = 0 -> output row i
                            acc[i][s0] = dw_add_lo(t.x, 0);
                            acc[i][s1] = dw_add_lo(t.z, acc[i][s1]);
                            acc[i][s2] = dw_add_hi(t.x, acc[i][s2]);
                        }
                        if (i >= 1 && i - 1 < R) {                     // ky = 1 -> output row i - 1
                            unsigned t11 = 0;
                            if (AXC_SHARED_OK(lane4 + qa * 128u, 4u, tab4, tab4 + kTab4Bytes, 302u))
                                asm("ld.shared.u32 %0, [%1];" : "=r"(t11) : "r"(lane4 + qa * 128u));
                            acc[i - 1][s0] = dw_add_lo(t.w, acc[i - 1][s0]);
                            acc[i - 1][s1] += int(t11);
                            acc[i - 1][s2] = dw_add_hi(t.w, acc[i - 1][s2]);
                        }
                        if (i >= 2) {                                  // ky = 2 -> output row i - 2
                            acc[i - 2][s0] = dw_add_lo(t.y, acc[i - 2][s0]);
                            acc[i - 2][s1] = dw_add_hi(t.z, acc[i - 2][s1]);
                            acc[i - 2][s2] = dw_add_hi(t.y, acc[i - 2][s2]);
                        }
                    }
                    if (TMA) tma_issue(c + STAGES, J);                 // the stage is free: every lane has used its taps
                    if (c >= 2) emit(c - 2, std::integral_constant<int, s2>{}, std::integral_constant<int, s1>{},
                                     std::integral_constant<int, s0>{}, std::integral_constant<int, s2>{});
                };
#pragma unroll
                for (int r = 0; r < R; ++r) { acc[r][1] = 0; acc[r][2] = 0; }
                if (TMA) {
#pragma unroll
                    for (int st = 0; st < STAGES; ++st) tma_issue(st, st);
                } else {
                    fetch(0);
                }
                const int c_end = P.OW + 2;
                for (int c = 0; c < c_end; c += 3) {
                    column(c, I0{});
                    if (c + 1 < c_end) column(c + 1, I1{});
                    if (c + 2 < c_end) column(c + 2, I2{});
                }
            } else {
                // even input column 2m: kx = 0 of output m and kx = 2 of output m - 1; odd column 2m + 1: kx = 1 of
                // output m.  Even input row 2r: ky = 0 of output row r and ky = 2 of row r - 1; odd row 2r + 1: ky = 1.
                auto even_column = [&](int m, auto jc) {
                    constexpr int J = decltype(jc)::value;            // m % 2
                    if (TMA) {
                        tma_take(I0{}, std::integral_constant<int, J>{});
                    } else {
#pragma unroll
                        for (int i = 0; i < IR; ++i) xf[i][J] = nx[i];
                        fetch(2 * m + 1);
                    }
#pragma unroll
                    for (int i = 0; i < IR; ++i) {
                        const unsigned qa = dw_q_u8(xf[i][J], in_off, in_inv);
                        if ((i & 1) == 0) {
                            unsigned tx = 0, ty = 0;
                            if (AXC_SHARED_OK(lane16 + qa * 512u, 8u, tab16, tab16 + kTab16Bytes, 303u))
                                asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(tx), "=r"(ty) : "r"(lane16 + qa * 512u));
                            if (i / 2 < R) {
                                acc[i / 2][J] = dw_add_lo(tx, 0);                                  // t00 starts the sum
                                acc[i / 2][J ^ 1] = dw_add_hi(tx, acc[i / 2][J ^ 1]);              // t02
                            }
                            if (i >= 2) {
                                acc[i / 2 - 1][J] = dw_add_lo(ty, acc[i / 2 - 1][J]);              // t20
                                acc[i / 2 - 1][J ^ 1] = dw_add_hi(ty, acc[i / 2 - 1][J ^ 1]);      // t22
                            }
                        } else {
                            unsigned tw = 0;
                            if (AXC_SHARED_OK(lane16 + qa * 512u + 12u, 4u, tab16, tab16 + kTab16Bytes, 304u))
                                asm("ld.shared.u32 %0, [%1];" : "=r"(tw) : "r"(lane16 + qa * 512u + 12u));
                            acc[i / 2][J] = dw_add_lo(tw, acc[i / 2][J]);                          // t10
                            acc[i / 2][J ^ 1] = dw_add_hi(tw, acc[i / 2][J ^ 1]);                  // t12
                        }
                    }
                    if (TMA) tma_issue(2 * m + STAGES, 0);
                    if (m >= 1) emit(m - 1, std::integral_constant<int, J ^ 1>{}, I2{}, std::integral_constant<int, J>{},
                                     std::integral_constant<int, J ^ 1>{});
                };
                auto odd_column = [&](int m, auto jc) {
                    constexpr int J = decltype(jc)::value;
                    if (TMA) {
                        tma_take(I1{}, I2{});
                    } else {
#pragma unroll
                        for (int i = 0; i < IR; ++i) xf[i][2] = nx[i];
                        fetch(2 * m + 2);
                    }
#pragma unroll
                    for (int i = 0; i < IR; ++i) {
                        const unsigned qa = dw_q_u8(xf[i][2], in_off, in_inv);
                        if ((i & 1) == 0) {
                            unsigned tz = 0;
                            if (AXC_SHARED_OK(lane16 + qa * 512u + 8u, 4u, tab16, tab16 + kTab16Bytes, 305u))
                                asm("ld.shared.u32 %0, [%1];" : "=r"(tz) : "r"(lane16 + qa * 512u + 8u));
                            if (i / 2 < R) acc[i / 2][J] = dw_add_lo(tz, acc[i / 2][J]);           // t01
                            if (i >= 2) acc[i / 2 - 1][J] = dw_add_hi(tz, acc[i / 2 - 1][J]);      // t21
                        } else {
                            unsigned t11 = 0;
                            if (AXC_SHARED_OK(lane4 + qa * 128u, 4u, tab4, tab4 + kTab4Bytes, 306u))
                                asm("ld.shared.u32 %0, [%1];" : "=r"(t11) : "r"(lane4 + qa * 128u));
                            acc[i / 2][J] += int(t11);
                        }
                    }
                    if (TMA) tma_issue(2 * m + 1 + STAGES, 1);
                };
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r][1] = 0;    // fed by column 0 for the output -1; output 1 initialises it
                if (TMA) {
#pragma unroll
                    for (int st = 0; st < STAGES; ++st) tma_issue(st, st);
                } else {
                    fetch(0);
                }
                for (int m = 0; m <= P.OW; m += 2) {
                    even_column(m, I0{});
                    if (m < P.OW) odd_column(m, I0{});
                    if (m + 1 <= P.OW) {
                        even_column(m + 1, I1{});
                        if (m + 1 < P.OW) odd_column(m + 1, I1{});
                    }
                }
            }
        }
    }
}

template <int S, int R, int NT, bool DBG>
__global__ void __launch_bounds__(NT, 1) depthwise_3x3_tab_kernel(const DwParams P)
{
    depthwise_3x3_tab_body<S, R, NT, DBG, false>(P, nullptr);
}

template <int S, int R, int NT, bool DBG>
__global__ void __launch_bounds__(NT, 1) depthwise_3x3_tma_kernel(const DwParams P, const __grid_constant__ CUtensorMap tmap)
{
    depthwise_3x3_tab_body<S, R, NT, DBG, true>(P, &tmap);
}

// Tiled tensor map of the NHWC input for boxes of (32 channels, 1 column, rows, 1 image); false when the
// tensor does not meet TMA's alignment rules (16-byte base and strides) or the driver entry point is missing.
bool dw_make_tensor_map(const DwParams &P, int rows, CUtensorMap *out)
{
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = []() -> encode_fn {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<encode_fn>(fn);
    }();
    if (!encode || P.C % 4 != 0 || (reinterpret_cast<uintptr_t>(P.input) & 15u) != 0) return false;
    const cuuint64_t dims[4] = {cuuint64_t(P.C), cuuint64_t(P.W), cuuint64_t(P.H), cuuint64_t(P.N)};
    const cuuint64_t strides[3] = {cuuint64_t(P.C) * 4, cuuint64_t(P.W) * P.C * 4, cuuint64_t(P.H) * P.W * P.C * 4};
    const cuuint32_t box[4] = {32, 1, cuuint32_t(rows), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(P.input), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int S, int R, int NT, bool DBG>
int launch_dw_tab_variant(DwParams P, const DeviceInfo &di, cudaStream_t stream)
{
    constexpr int IR = (R - 1) * S + 3;
    constexpr int STAGES = S == 1 ? 3 : 2;
    P.bands = (P.OH + R - 1) / R;
    P.units_per_group = P.N * P.bands;
    P.wave = P.groups < di.sm_count ? P.groups : di.sm_count;
    P.sets = di.sm_count / P.wave;
    if (P.sets > P.units_per_group) P.sets = P.units_per_group;
    // Input columns by TMA where the tensor allows it (at least 32 channels, and a channel multiplier of 1, so that
    // a lane's input channel is its output channel); plain loads otherwise.
    CUtensorMap tmap;
    const unsigned tma_smem = kTabSmem + unsigned(NT / 32 * STAGES) * (unsigned(IR) * 128u + 8u);
    if (P.mult == 1 && P.C >= 32 && tma_smem <= unsigned(di.max_smem_optin) && dw_make_tensor_map(P, IR, &tmap)) {
        AXC_CUDA(cudaFuncSetAttribute(depthwise_3x3_tma_kernel<S, R, NT, DBG>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(tma_smem)));
        depthwise_3x3_tma_kernel<S, R, NT, DBG><<<unsigned(P.wave * P.sets), NT, tma_smem, stream>>>(P, tmap);
        AXC_CUDA(cudaGetLastError());
        count_launch();
        return AXC_OK;
    }
    AXC_CUDA(cudaFuncSetAttribute(depthwise_3x3_tab_kernel<S, R, NT, DBG>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kTabSmem)));
    depthwise_3x3_tab_kernel<S, R, NT, DBG><<<unsigned(P.wave * P.sets), NT, kTabSmem, stream>>>(P);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    return AXC_OK;
}

template <int S, int R, int NT>
int launch_dw_tab(const DwParams &P, const DeviceInfo &di, cudaStream_t stream)
{
    if (P.acc_out) return launch_dw_tab_variant<S, R, NT, true>(P, di, stream);
    return launch_dw_tab_variant<S, R, NT, false>(P, di, stream);
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
    // the register-window and generic kernels keep the table at the window addresses 64 KiB .. 192 KiB
    if (di.max_smem_optin < int(kSmemEnd) || di.smem_base > kLutBase || di.smem_end < kSmemEnd) return AXC_INTERNAL;
    const int OC = g.C * g.Cout;
    const Workspace ws = depthwise_workspace(g.K, g.C, g.Cout);
    unsigned char *wsb = static_cast<unsigned char *>(workspace);
    uint32_t *prog = reinterpret_cast<uint32_t *>(wsb);
    uint32_t *prog_packed = prog + size_t(g.K) * OC;
    float *bsum = reinterpret_cast<float *>(wsb + ws.sums_off);
    int *status = reinterpret_cast<int *>(wsb + ws.status_off);

    dw_filter_prep_kernel<<<unsigned((OC + 127) / 128), 128, 0, stream>>>(filter, g.K, OC, q.f_off, q.f_inv, prog, prog_packed,
                                                                         bsum, dbg ? dbg->qfilter : nullptr, status);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    if (dbg && dbg->qinput) {
        const long long n = (long long)g.N * g.H * g.W * g.C;
        if (n > 0) {
            const unsigned blocks = unsigned(n / 256 + 1 < 4096 ? n / 256 + 1 : 4096);
            dw_quantize_tensor_kernel<<<blocks, 256, 0, stream>>>(input, n, q.in_off, q.in_inv, dbg->qinput, g.ep.input_relu ? 0.0f : -INFINITY);
            AXC_CUDA(cudaGetLastError());
            count_launch();
        }
    }

    DwParams P;
    P.lut = lut_dev; P.input = input; P.output = output; P.prog = prog; P.prog_packed = prog_packed; P.bsum = bsum;
    P.acc_out = dbg ? dbg->acc : nullptr;
    P.status = status;
    P.N = g.N; P.H = g.H; P.W = g.W; P.C = g.C; P.KH = g.KH; P.KW = g.KW; P.mult = g.Cout; P.OC = OC;
    P.sh = g.sh; P.sw = g.sw; P.dh = g.dh; P.dw = g.dw; P.ph = g.ph; P.pw = g.pw; P.OH = g.OH; P.OW = g.OW;
    P.run = g.OW < 15 ? g.OW : 15;   // a multiple of the 3x3 kernels' batch of three outputs
    P.runs_per_row = (g.OW + P.run - 1) / P.run;
    P.groups = (OC + 31) / 32;
    P.items = (long long)g.N * g.OH * P.runs_per_row * P.groups;
    P.in_off = q.in_off; P.in_inv = q.in_inv; P.s1s2 = q.s1s2; P.m1 = q.m1; P.m2 = q.m2;
    {
        volatile float kf = float(g.K);
        volatile float t3 = kf * q.m1m2;
        P.km1m2 = t3;
    }
    const bool small = (long long)g.N * g.H * g.W * g.C < (1ll << 31) && g.M * OC < (1ll << 31) && P.items < (1ll << 31);
    const bool k3 = small && g.KH == 3 && g.KW == 3 && g.dh == 1 && g.dw == 1 && g.sh == g.sw;
    P.filter = filter; P.f_off = q.f_off; P.f_inv = q.f_inv;
    P.bands = 0; P.units_per_group = 0; P.wave = 0; P.sets = 0;
    P.ep = g.ep;
    P.in_floor = g.ep.input_relu ? 0.0f : -INFINITY;
    // The expanded-table kernel pays about 74 000 lookups per CTA and channel group for its table: worth it from
    // some ten thousand outputs per group on.
    if (k3 && (g.sw == 1 || g.sw == 2) && g.M * 32 >= kTabMinOutputsPerGroup && di.max_smem_optin >= int(kTabSmem) &&
        (long long)g.W * g.C * 4 * 16 < (1ll << 32) && (long long)g.OW * OC * 4 * 8 < (1ll << 32)) {
        if (g.sw == 1) return launch_dw_tab<1, 7, 512>(P, di, stream);
        return launch_dw_tab<2, 4, 512>(P, di, stream);
    }
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

AXC_DEFINE_BOUNDS_READER(bounds_record_depthwise)

int depthwise_status(const Geom &g, const void *workspace, int32_t *status, int device, cudaStream_t stream)
{
    const Workspace ws = depthwise_workspace(g.K, g.C, g.Cout);
    int prev = 0;
    AXC_CUDA(cudaGetDevice(&prev));
    if (prev != device) AXC_CUDA(cudaSetDevice(device));
    int rc = AXC_OK;
    const void *base = workspace;
    if (!base) {
        if (ws.total > kStaticScratchBytes) rc = AXC_INVALID_ARGUMENT;
        void *p = nullptr;
        if (rc == AXC_OK) rc = static_scratch_address(device, &p);
        base = p;
    }
    cudaError_t e = cudaSuccess;
    if (rc == AXC_OK) e = cudaStreamSynchronize(stream);
    if (rc == AXC_OK && e == cudaSuccess)
        e = cudaMemcpy(status, static_cast<const unsigned char *>(base) + ws.status_off, sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_failed(e);
    return rc;
}

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
