// Bank-scheduled dense table convolution for sm_100a.
//
// Why: with lanes = output channels and all lanes on the same K index, the 32 table lookups of a
// warp instruction hit the 32 shared-memory banks at random (the bank of LUT[a][b] is a function of the
// weight b alone), which costs about 2.1 wavefronts per instruction.  Integer accumulation is exact and
// commutative, so every lane may walk its K elements in its own order.  For each group of 32 output
// channels and each K chunk a schedule is built (once per filter, kept in the caller's workspace) in which,
// at every step, the 32 lanes look up 32 different banks: a step is one conflict-free wavefront per pixel.
//
//   plan_check_kernel   quantise the filter, compare with the stored copy -> `dirty`
//   plan_sigma_kernel   column permutation sigma of the table (8 columns per bank): spreads the weight histogram
//                       over the 32 banks, then lowers the heaviest bank of every (group, chunk) by local search
//   plan_build_kernel   per (channel group, chunk): the schedule.  The two lanes of a pair (2p, 2p+1) always work
//                       on the same K element, so that they fetch the same activation row; also the permuted
//                       table image and the sequential per-channel filter sums
//   dense_sched_kernel  the convolution: 16 pixels per tile; a lane fetches the 16 activation bytes of "its" K row
//                       with one LDS.128 (2 pipe cycles because neighbouring lanes share the address and the 8
//                       rows of a half warp lie in different bank groups), then 16 x (PRMT, LDS.U16, IADD)
//
// Arithmetic (quantiser, table index, dequantisation) is the reference's,
// tf2/src/approx_nn_conv_kernels.cpp:167-296; results are bit-identical to the common-K kernel.
#include <cmath>

#include "axc_internal.h"
#include "axc_sched.h"
#include <vector>

namespace axc {

namespace {

constexpr unsigned kLutBase = 65536u;          // table planes at 64 KiB and 128 KiB
constexpr unsigned kBuf1Base = 196608u;        // 32 zero words (one per bank), then activation buffers
constexpr unsigned kWindowEnd = 233472u;       // 228 KiB shared window of an SM
constexpr int kComputeWarps = 8;
// loader warps per CTA: 4 (168 registers per thread), or 8 for launches of one channel group, whose loaders
// otherwise cannot keep up (each activation byte then serves only 32 or 16 output channels)
constexpr int kTilePix = 16;
constexpr int kTapTableMax = 512;
constexpr int kStepsInSmemMax = 1024;
constexpr uint32_t kPlanMagic = 0x41584334u;   // "AXC4"

__device__ __forceinline__ unsigned q_u8(float x, float off, float inv)
{
    const float v = __fadd_rn(__fmul_rn(__fsub_rn(x, off), inv), 0.5f);
    unsigned u;
    asm("cvt.rzi.u8.f32 %0, %1;" : "=r"(u) : "f"(v));     // truncates and clamps to 0..255 (NaN -> 0)
    return u;
}

// prmt.b32 with an immediate selector; a selector nibble with bit 3 set replicates the sign of the byte
template <unsigned SEL>
__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b)
{
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "n"(SEL));
    return d;
}

// the same with the selector in a register
__device__ __forceinline__ unsigned prmt_r(unsigned a, unsigned b, unsigned sel)
{
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Shared-memory accessors.  In the debug flavour each checks its address first (table lookups: the two table planes
// and the zero words; everything else: the CTA's window) and skips the access on a violation.
__device__ __forceinline__ unsigned lds16(unsigned addr)
{
    if (!AXC_SHARED_OK(addr, 2u, kLutBase, kBuf1Base + 128u, 101u)) return 0u;
    unsigned v;
    asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(unsigned addr)
{
    if (!AXC_SHARED_OK(addr, 16u, 0u, kWindowEnd, 102u)) return make_uint4(0, 0, 0, 0);
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(unsigned addr, uint4 v)
{
    if (!AXC_SHARED_OK(addr, 16u, 0u, kWindowEnd, 103u)) return;
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts8(unsigned addr, unsigned v)
{
    if (!AXC_SHARED_OK(addr, 1u, 0u, kWindowEnd, 104u)) return;
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts32(unsigned addr, unsigned v)
{
    if (!AXC_SHARED_OK(addr, 4u, 0u, kWindowEnd, 105u)) return;
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned lds32(unsigned addr)
{
    if (!AXC_SHARED_OK(addr, 4u, 0u, kWindowEnd, 106u)) return 0u;
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ int slot_bank(int s) { return ((s & 127) >> 1) & 31; }

// ------------------------------------------------------------------------------------------------
// plan_check: quantisation parameters of the call, quantised filter vs. stored copy, structure of the stored plan
// ------------------------------------------------------------------------------------------------
// Range nudging on the device, operation by operation as on the host (axc_api.cu var_quant_props).
__device__ void dev_var_quant(float min_v, float max_v, float *scale, float *inv, float *offset)
{
    float s = 0.0f, i = 0.0f, nudged_min = 0.0f;
    if (min_v != 0.0f || max_v != 0.0f) {
        s = __fdiv_rn(__fsub_rn(max_v, min_v), 255.0f);
        const float zp_from_min = __fsub_rn(0.0f, __fdiv_rn(min_v, s));
        float zp;
        if (zp_from_min < 0.0f) zp = 0.0f;
        else if (zp_from_min > 255.0f) zp = 255.0f;
        else zp = roundf(zp_from_min);                       // half away from zero, like std::round
        nudged_min = __fmul_rn(__fsub_rn(0.0f, zp), s);      // a true subtraction: +0.0 for zp == 0
        i = __fdiv_rn(1.0f, s);
    }
    *scale = s; *inv = i; *offset = nudged_min;
}

__device__ DevQuant dev_quant_from_ranges(const float *__restrict__ ranges, int K)
{
    float s1, i1, o1, s2, i2, o2;
    dev_var_quant(ranges[0], ranges[1], &s1, &i1, &o1);
    dev_var_quant(ranges[2], ranges[3], &s2, &i2, &o2);
    DevQuant q;
    q.in_off = o1; q.in_inv = i1; q.f_off = o2; q.f_inv = i2;
    q.s1s2 = __fmul_rn(s1, s2); q.m1 = o1; q.m2 = o2;
    q.km1m2 = __fmul_rn(float(K), __fmul_rn(o1, o2));
    return q;
}

// A program word is safe to execute when the shared-memory addresses the kernel forms from it stay inside the
// table planes, the zero words and the activation buffers, and are aligned: plane byte 1 or 2 with an even column
// byte, or the idle form (plane byte 3, bit 14 set, column byte a multiple of 4 below 128); activation row offset a
// multiple of 16 and at most 16 * (KC + 7).
__device__ __forceinline__ bool prog_word_ok(uint32_t w, int KC)
{
    const unsigned col = w & 0xFFu, plane = (w >> 16) & 0xFFu, idle = (w >> 14) & 1u;
    const unsigned rowoff = (w >> 24) | (w & 0x3F00u);
    const bool lookup_ok = idle ? (plane == 3u && (col & 3u) == 0u && col < 128u) : ((plane == 1u || plane == 2u) && (col & 1u) == 0u);
    return lookup_ok && (w & 0x8000u) == 0u && (rowoff & 15u) == 0u && rowoff <= 16u * unsigned(KC + 7);
}

// Every call: (1) block 0 writes the quantisation parameters of the call into the workspace - `host_q`, or derived
// from the four range scalars in device memory; (2) the filter is quantised and compared with the stored copy;
// (3) the stored plan is checked structurally - header, step counts within their reserve, every program word that
// the convolution would execute (prog_word_ok) - so that a buffer whose tail was overwritten by someone else can
// give wrong numbers at worst, never an access outside shared memory or the workspace: it is rebuilt instead.
// A plan found wanting gets `dirty` and loses its magic word until plan_build has finished the new one.
__global__ void plan_check_kernel(const float *__restrict__ filter, long long count, DevQuant host_q,
                                  const float *__restrict__ ranges, int K, unsigned char *__restrict__ plan, PlanLayout L,
                                  uint8_t *__restrict__ qf_debug, PlanHeader want)
{
    PlanHeader *hdr = reinterpret_cast<PlanHeader *>(plan);
    uint8_t *qf = plan + L.qf_off;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    const DevQuant q = ranges ? dev_quant_from_ranges(ranges, K) : host_q;
    const float f_off = q.f_off, f_inv = q.f_inv;
    bool bad = false;
    if (idx == 0) {
        *reinterpret_cast<DevQuant *>(plan + kDevQuantOffset) = q;
        bad = !(hdr->magic == want.magic && hdr->K == want.K && hdr->Cout == want.Cout && hdr->G == want.G &&
                hdr->NCH == want.NCH && hdr->KC == want.KC && hdr->sqcap == want.sqcap &&
                hdr->table_uid == want.table_uid && hdr->f_off_bits == __float_as_uint(f_off) &&
                hdr->f_inv_bits == __float_as_uint(f_inv));
        hdr->status = 0;
    }
    if (idx < count) {
        const unsigned b = q_u8(filter[idx], f_off, f_inv);
        if (qf[idx] != b) {
            qf[idx] = uint8_t(b);
            bad = true;
        }
        if (qf_debug) qf_debug[idx] = uint8_t(b);
    }
    // structure of the stored plan
    const int n_sched = L.G * L.NCH;
    const int *steps = reinterpret_cast<const int *>(plan + L.steps_off);
    for (long long e = idx; e < n_sched; e += nthreads) bad |= unsigned(steps[e]) > unsigned(L.sqcap);
    const uint4 *prog = reinterpret_cast<const uint4 *>(plan + L.prog_off);
    const long long quads = (long long)n_sched * L.sqcap * 32;
    for (long long e = idx; e < quads; e += nthreads) {
        const long long row = e >> 5;
        const int sc = int(row / L.sqcap), qi = int(row - (long long)sc * L.sqcap);
        if (unsigned(qi) < unsigned(steps[sc])) {
            const uint4 w = prog[e];
            bad |= !(prog_word_ok(w.x, L.KC) && prog_word_ok(w.y, L.KC) && prog_word_ok(w.z, L.KC) && prog_word_ok(w.w, L.KC));
        }
    }
    if (bad) {
        hdr->magic = 0;
        atomicOr(&hdr->dirty, 1);
    }
}

// ------------------------------------------------------------------------------------------------
// plan_sigma: assignment of the 256 table columns to the 32 banks (8 columns per bank).
//  1. histogram of the quantised weights; largest column first into the bank with the smallest mass that still
//     has a free slot: balances the banks over the whole filter;
//  2. local search on the blocks the schedules are built for ((32 channels) x (K chunk)): a schedule cannot be
//     shorter than the heaviest bank of its block, so columns are swapped between banks while that lowers the
//     sum over blocks of max(heaviest bank, the block's own lower bound).  Deterministic.
// One block of 256 threads; dynamic shared memory: per block 128 words of packed 16-bit column counts and 32
// words of bank loads (skipped when that does not fit).
// ------------------------------------------------------------------------------------------------
constexpr int kSigmaMaxBlocks = 320;
constexpr int kSigmaIters = 600;

__global__ void __launch_bounds__(256) plan_sigma_kernel(const uint8_t *__restrict__ qf, int K, int Cout, PlanLayout L,
                                                         int search_blocks, uint8_t *__restrict__ sigma, PlanHeader *hdr,
                                                         PlanHeader want, const DevQuant *__restrict__ dq)
{
    if (hdr->dirty == 0) return;
    if (threadIdx.x == 0) hdr->blocks_done = 0;
    extern __shared__ __align__(16) unsigned sigma_smem[];
    __shared__ unsigned hist[256];
    __shared__ int value_at_rank[256];
    __shared__ unsigned long long mass[32];
    __shared__ int used[32];
    __shared__ unsigned char bank_of[256];
    __shared__ long long red_key[8];
    __shared__ int s_target, s_b1, s_done;
    const int t = threadIdx.x;
    const long long count = (long long)K * Cout;
    hist[t] = 0;
    __syncthreads();
    for (long long i = t; i < count; i += 256) atomicAdd(&hist[qf[i]], 1u);
    __syncthreads();
    {
        const unsigned h = hist[t];
        int rank = 0;
        for (int u = 0; u < 256; ++u) {
            const unsigned hu = hist[u];
            rank += (hu > h || (hu == h && u < t)) ? 1 : 0;
        }
        value_at_rank[rank] = t;
    }
    if (t < 32) { mass[t] = 0; used[t] = 0; }
    __syncthreads();
    if (t < 32) {
        for (int r = 0; r < 256; ++r) {
            const int v = value_at_rank[r];
            // bank with the smallest mass among those with a free slot; ties -> lowest bank
            unsigned long long key = used[t] < 8 ? ((mass[t] << 5) | (unsigned long long)t) : ~0ull;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
                key = other < key ? other : key;
            }
            const int bank = int(key & 31ull);
            if (t == bank) {
                bank_of[v] = (unsigned char)bank;
                used[t]++;
                mass[t] += hist[v];
            }
            __syncwarp();
        }
    }
    __syncthreads();

    const int B = search_blocks;                       // 0: no local search
    if (B > 0) {
        unsigned *H = sigma_smem;                      // [B][128]: counts of columns 2i, 2i+1 in the halves of word i
        int *Ld = reinterpret_cast<int *>(H + (size_t)B * 128);   // [B][32] bank loads
        int *top = Ld + (size_t)B * 32;                // [B][4]: the three largest loads packed {load:26, bank:5}, then the floor
        for (int i = t; i < B * 128; i += 256) H[i] = 0;
        __syncthreads();
        const int NCH = L.NCH, KC = L.KC;
        for (long long i = t; i < count; i += 256) {
            const int l = int(i / Cout), j = int(i - (long long)l * Cout);
            const int blk = (j >> 5) * NCH + l / KC;
            const unsigned v = qf[i];
            atomicAdd(&H[blk * 128 + (v >> 1)], 1u << (16 * (v & 1u)));
        }
        __syncthreads();
        auto h_at = [&](int blk, int v) -> int { return int((H[blk * 128 + (v >> 1)] >> (16 * (v & 1))) & 0xFFFFu); };
        for (int i = t; i < B * 32; i += 256) {
            const int blk = i >> 5, b = i & 31;
            int sum = 0;
            for (int v = 0; v < 256; ++v) sum += bank_of[v] == b ? h_at(blk, v) : 0;
            Ld[i] = sum;
        }
        __syncthreads();
        for (int i = t; i < B; i += 256) {
            // lower bound of the block's schedule that no column assignment changes: its K elements plus the
            // share that ends up split (two weights of a lane pair in one bank), about 1/32
            const int c = i % NCH;
            const int kc = min(KC, K - c * KC);
            top[i * 4 + 3] = kc + (kc >> 5);
        }
        if (t == 0) s_done = 0;
        __syncthreads();
        for (int iter = 0; iter < kSigmaIters; ++iter) {
            // the three heaviest banks of every block
            for (int i = t; i < B; i += 256) {
                int a0 = -1, a1 = -1, a2 = -1;
                for (int b = 0; b < 32; ++b) {
                    const int key = (Ld[i * 32 + b] << 5) | b;
                    if (key > a0) { a2 = a1; a1 = a0; a0 = key; }
                    else if (key > a1) { a2 = a1; a1 = key; }
                    else if (key > a2) a2 = key;
                }
                top[i * 4 + 0] = a0; top[i * 4 + 1] = a1; top[i * 4 + 2] = a2;
            }
            __syncthreads();
            // target: the block that exceeds its floor the most (flagged blocks excluded); ties -> lowest block
            {
                long long key = -1;
                for (int i = t; i < B; i += 256) {
                    const int fl = top[i * 4 + 3];
                    if (fl < 0) continue;                                  // flagged: no improving swap last time
                    const int ex = (top[i * 4 + 0] >> 5) - fl;
                    if (ex > 0) { const long long k2 = ((long long)ex << 20) | (long long)(0xFFFFF - i); key = k2 > key ? k2 : key; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) { const long long other = __shfl_xor_sync(0xffffffffu, key, o); key = other > key ? other : key; }
                if ((t & 31) == 0) red_key[t >> 5] = key;
                __syncthreads();
                if (t == 0) {
                    long long best = -1;
                    for (int w = 0; w < 8; ++w) best = red_key[w] > best ? red_key[w] : best;
                    if (best < 0) s_done = 1;
                    else { s_target = 0xFFFFF - int(best & 0xFFFFF); s_b1 = top[s_target * 4 + 0] & 31; }
                }
                __syncthreads();
            }
            if (s_done) break;
            const int target = s_target, b1 = s_b1;
            // candidate swaps: a column of bank b1 against column t of another bank; change of the objective
            long long best_key = 0;                     // {-(delta) : 32, v1 : 8, v2 : 8}, 0 = none
            const int b2 = bank_of[t];
            if (b2 != b1) {
                for (int v1 = 0; v1 < 256; ++v1) {
                    if (bank_of[v1] != b1) continue;
                    int delta = 0;
                    for (int i = 0; i < B; ++i) {
                        const int d = h_at(i, v1) - h_at(i, t);
                        if (d == 0) continue;
                        const int fl = top[i * 4 + 3] & 0x7FFFFFFF;
                        const int k0 = top[i * 4 + 0], k1 = top[i * 4 + 1], k2 = top[i * 4 + 2];
                        // heaviest bank other than b1 and b2
                        int others = ((k0 & 31) != b1 && (k0 & 31) != b2) ? (k0 >> 5) : ((k1 & 31) != b1 && (k1 & 31) != b2) ? (k1 >> 5) : (k2 >> 5);
                        const int n1 = Ld[i * 32 + b1] - d, n2 = Ld[i * 32 + b2] + d;
                        const int new_max = max(others, max(n1, n2));
                        delta += max(new_max, fl) - max(k0 >> 5, fl);
                    }
                    if (delta < 0) {
                        const long long key = ((long long)(-delta) << 16) | (long long)((255 - v1) << 8) | (long long)(255 - t);
                        best_key = key > best_key ? key : best_key;
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { const long long other = __shfl_xor_sync(0xffffffffu, best_key, o); best_key = other > best_key ? other : best_key; }
            if ((t & 31) == 0) red_key[t >> 5] = best_key;
            __syncthreads();
            long long best = 0;
            for (int w = 0; w < 8; ++w) best = red_key[w] > best ? red_key[w] : best;
            __syncthreads();
            if (best == 0) {
                if (t == 0) top[target * 4 + 3] |= int(0x80000000u);      // flag: leave this block alone
                __syncthreads();
                continue;
            }
            const int v1 = 255 - int((best >> 8) & 255), v2 = 255 - int(best & 255);
            const int bb2 = bank_of[v2];
            __syncthreads();
            for (int i = t; i < B; i += 256) {
                const int d = h_at(i, v1) - h_at(i, v2);
                Ld[i * 32 + b1] -= d;
                Ld[i * 32 + bb2] += d;
                top[i * 4 + 3] &= 0x7FFFFFFF;                              // loads changed: every block is eligible again
            }
            if (t == 0) { bank_of[v1] = (unsigned char)bb2; bank_of[v2] = (unsigned char)b1; }
            __syncthreads();
        }
    }
    __syncthreads();
    // slots: the 8 columns of a bank in increasing order; slot = word bank or bank+32 of a plane row, low/high
    // half, plane 0/1
    {
        const int bank = bank_of[t];
        int k = 0;
        for (int v = 0; v < t; ++v) k += bank_of[v] == bank ? 1 : 0;
        const int slot = (k >> 2) * 128 + 2 * (bank + 32 * ((k >> 1) & 1)) + (k & 1);
        sigma[t] = uint8_t(slot);
    }
    if (t == 0) {
        // the magic word is written by the last block of plan_build: a plan is valid only once it is complete
        hdr->K = want.K; hdr->Cout = want.Cout; hdr->G = want.G; hdr->NCH = want.NCH;
        hdr->KC = want.KC; hdr->sqcap = want.sqcap; hdr->table_uid = want.table_uid;
        hdr->f_off_bits = __float_as_uint(dq->f_off); hdr->f_inv_bits = __float_as_uint(dq->f_inv);
        hdr->fallback = 0;
    }
}

// ------------------------------------------------------------------------------------------------
// plan_build.  blockIdx.x < G*NCH: schedule of (group, chunk), one warp.  Then 256 blocks that write the
// permuted table image, then ceil(Cout/32) blocks for the filter sums.
//
// A step assigns to every lane pair (= two neighbouring output channels of the group) one K element of the
// chunk such that
//   (1) the table columns looked up by the 32 lanes lie in 32 different banks,
//   (2) both lanes of the pair read the same activation row (16 bytes, one LDS.128), and
//   (3) the 8 rows read by a half warp lie in 8 different 16-byte bank groups, i.e. have different (row mod 8).
// An element whose two weights fall into the same bank is split: each lane does it in a step of its own while
// its neighbour idles on the same row.  Greedy: pairs with the most work left first, each taking the admissible
// item with the heaviest banks; then a repair pass (see the loop).  Idle lanes look up one of 32 zero words (one
// per bank); bit 14 of their program word makes the kernel put 0 in place of the activation byte, whatever row
// they read; a pair without an item reads one of 8 all-zero rows (one per row class).
//
// Program word of a step:  byte0 = 2*(slot&127)  byte2 = 1 + (slot>>7)   {byte1:byte3} = 16 * row
// with row = 8 + (l - chunk start); idle: byte0 = 4*bank, byte2 = 3, bit 14 set.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) plan_build_kernel(const float *__restrict__ filter, const uint16_t *__restrict__ lut,
                                                        unsigned char *__restrict__ plan, PlanLayout L, int K, int Cout)
{
    PlanHeader *hdr = reinterpret_cast<PlanHeader *>(plan);
    if (hdr->dirty == 0) return;
    const uint8_t *qf = plan + L.qf_off;
    const uint8_t *sigma = plan + L.sigma_off;
    const int lane = threadIdx.x;
    const int n_sched = L.G * L.NCH;
    // the block that finishes last seals the plan
    auto block_done = [&]() {
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            if (atomicAdd(&hdr->blocks_done, 1) == int(gridDim.x) - 1) {
                __threadfence();
                hdr->magic = kPlanMagic;
            }
        }
    };

    if (int(blockIdx.x) >= n_sched) {
        const int rest = int(blockIdx.x) - n_sched;
        if (rest < 256) {
            // table image: plane p = slot>>7 at p*65536, row a at a*256, column 2*(slot&127)
            const int a = rest;
            uint16_t *img = reinterpret_cast<uint16_t *>(plan + L.lut_off);
            for (int b = lane; b < 256; b += 32) {
                const int s = sigma[b];
                img[((s >> 7) * 65536 + a * 256 + 2 * (s & 127)) >> 1] = lut[a * 256 + b];
            }
        } else {
            // filter sums in l order (tf2/src/approx_nn_conv_kernels.cpp:187-197)
            const int j = (rest - 256) * 32 + lane;
            if (j < Cout) {
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
                reinterpret_cast<float *>(plan + L.bsum_off)[j] = acc;
            }
        }
        block_done();
        return;
    }

    // Items of the 16 lane pairs, packed {k:10, bank:5, bank2:5, kind:2}.  kind 0: both lanes look up row k
    // (banks bank / bank2); kind 1 / 2: only the even / odd lane does (its bank in `bank`), the other lane idles
    // on the same row.  A K element whose two weights fall into the same bank becomes one item of each kind.
    extern __shared__ __align__(16) unsigned char sched_smem[];
    const int cap = 2 * L.KC;
    uint32_t *items = reinterpret_cast<uint32_t *>(sched_smem);               // [16][cap]
    __shared__ int cnt[16], pick[16], order[16], own_cls[16], load[32], own_bank[32];

    const int g = int(blockIdx.x) / L.NCH, c = int(blockIdx.x) % L.NCH;
    const int l_base = c * L.KC;
    const int kc = min(L.KC, K - l_base);
    // at most 16 live channels in a group launched alone: the two half warps carry the same channels (for two
    // different pixel tiles)
    const bool dual = plan_group_dual(g, L.G, Cout, K);
    auto channel_of = [&](int ln) { return g * 32 + (dual ? (ln & 15) : ln); };
    auto bank_of = [&](int k, int j) { return slot_bank(sigma[qf[(size_t)(l_base + k) * Cout + j]]); };
    auto item_banks = [](uint32_t it) -> unsigned {
        return (1u << ((it >> 10) & 31u)) | (((it >> 20) & 3u) == 0u ? (1u << ((it >> 15) & 31u)) : 0u);
    };

    load[lane] = 0;
    if (lane < 16) cnt[lane] = 0;
    __syncwarp();
    int total = 0;
    for (int p = 0; p < 16; ++p) {
        const int ja = channel_of(2 * p), jb = channel_of(2 * p + 1);
        const bool la = ja < Cout, lb = jb < Cout;
        int n_pair = 0;
        for (int k0 = 0; k0 < kc; k0 += 32) {
            const int k = k0 + lane;
            uint32_t it0 = 0, it1 = 0;
            int n = 0;
            if (k < kc && (la || lb)) {
                const int ba = la ? bank_of(k, ja) : 0, bb = lb ? bank_of(k, jb) : 0;
                if (la && lb && ba != bb) { it0 = uint32_t(k) | (uint32_t(ba) << 10) | (uint32_t(bb) << 15); n = 1; }
                else {
                    if (la) { it0 = uint32_t(k) | (uint32_t(ba) << 10) | (1u << 20); n = 1; }
                    if (lb) { const uint32_t t = uint32_t(k) | (uint32_t(bb) << 10) | (2u << 20); if (n) it1 = t; else it0 = t; ++n; }
                }
            }
            int pre = n;                                // inclusive scan over the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, pre, o); if (lane >= o) pre += v; }
            const int at = n_pair + pre - n;
            if (n > 0) { items[p * cap + at] = it0; atomicAdd(&load[(it0 >> 10) & 31u], 1); if (((it0 >> 20) & 3u) == 0u) atomicAdd(&load[(it0 >> 15) & 31u], 1); }
            if (n > 1) { items[p * cap + at + 1] = it1; atomicAdd(&load[(it1 >> 10) & 31u], 1); }
            n_pair += __shfl_sync(0xffffffffu, pre, 31);
        }
        if (lane == 0) cnt[p] = n_pair;
        total += n_pair;
    }
    __syncwarp();

    // best admissible item of pair p: banks free in `used`, row class free in `cls` (the pair's half warp);
    // heaviest banks first.  Returns the item index or -1 (the same value in every lane).
    auto scan_best = [&](int p, unsigned used, unsigned cls) -> int {
        const int n = cnt[p];
        unsigned best = 0;
        for (int i = lane; i < n; i += 32) {
            const uint32_t it = items[p * cap + i];
            if ((cls >> (it & 7u)) & 1u) continue;
            if (used & item_banks(it)) continue;
            const int l1 = load[(it >> 10) & 31u];
            const int l2 = ((it >> 20) & 3u) == 0u ? load[(it >> 15) & 31u] : l1;
            const unsigned key = (unsigned(l1 + l2) << 12) | unsigned(4095 - i);
            best = key > best ? key : best;
        }
        best = __reduce_max_sync(0xffffffffu, best);
        return best == 0u ? -1 : 4095 - int(best & 4095u);
    };
    // book-keeping of one choice (sign = +1 take, -1 give back); every lane calls it with the same arguments
    auto account = [&](int p, uint32_t it, int sign) {
        if (lane == 0) {
            const int b1 = (it >> 10) & 31u, b2 = (it >> 15) & 31u;
            const bool both = ((it >> 20) & 3u) == 0u;
            own_bank[b1] = sign > 0 ? p : -1;
            load[b1] -= sign;
            if (both) { own_bank[b2] = sign > 0 ? p : -1; load[b2] -= sign; }
            own_cls[(p >> 3) * 8 + int(it & 7u)] = sign > 0 ? p : -1;
        }
        __syncwarp();
    };

    uint4 *prog = reinterpret_cast<uint4 *>(plan + L.prog_off) + (size_t)blockIdx.x * L.sqcap * 32;
    const int step_cap = L.sqcap * 4;
    const int my_pair = lane >> 1, side = lane & 1, my_half = lane >> 4;
    const int j = channel_of(lane);
    uint32_t wq[4] = {0, 0, 0, 0};
    int step = 0;
    bool overflow = false;
    while (total > 0) {
        if (step >= step_cap) { overflow = true; break; }
        own_bank[lane] = -1;
        if (lane < 16) {
            own_cls[lane] = -1;
            pick[lane] = -1;
            const int mine = cnt[lane];
            int rank = 0;
            for (int x = 0; x < 16; ++x) { const int cx = cnt[x]; rank += (cx > mine || (cx == mine && x < lane)) ? 1 : 0; }
            order[rank] = lane;
        }
        __syncwarp();
        unsigned used = 0, cls[2] = {0, 0};
        // greedy pass: pairs with the most items left choose first
        for (int r = 0; r < 16; ++r) {
            const int p = order[r];
            if (cnt[p] == 0) break;
            const int idx = scan_best(p, used, cls[p >> 3]);
            if (idx < 0) continue;
            const uint32_t it = items[p * cap + idx];
            if (lane == 0) pick[p] = idx;
            used |= item_banks(it);
            cls[p >> 3] |= 1u << (it & 7u);
            account(p, it, +1);
        }
        // repair pass: a pair left without an item takes one that a single other pair blocks, if that pair can
        // move to another of its items
        for (int r = 0; r < 16; ++r) {
            const int p = order[r];
            const int n = cnt[p];
            if (n == 0) break;
            if (pick[p] >= 0) continue;
            const int h = p >> 3;
            bool found = false;
            int tries = 0;
            for (int base = 0; base < n && !found && tries < 6; base += 32) {
                const int i = base + lane;
                uint32_t it = 0;
                int q = -2;                                  // -2: not a candidate
                if (i < n) {
                    it = items[p * cap + i];
                    const int o1 = own_bank[(it >> 10) & 31u];
                    const int o2 = ((it >> 20) & 3u) == 0u ? own_bank[(it >> 15) & 31u] : -1;
                    const int o3 = own_cls[h * 8 + int(it & 7u)];
                    const int m = max(o1, max(o2, o3));
                    if ((o1 < 0 || o1 == m) && (o2 < 0 || o2 == m) && (o3 < 0 || o3 == m)) q = m;   // -1: free as it is
                }
                unsigned mask = __ballot_sync(0xffffffffu, q > -2);
                while (mask != 0u && !found && tries < 6) {
                    const int src = __ffs(int(mask)) - 1;
                    mask &= mask - 1u;
                    ++tries;
                    const uint32_t itc = __shfl_sync(0xffffffffu, it, src);
                    const int qq = __shfl_sync(0xffffffffu, q, src);
                    if (qq < 0) {
                        if (lane == 0) pick[p] = base + src;
                        used |= item_banks(itc);
                        cls[h] |= 1u << (itc & 7u);
                        account(p, itc, +1);
                        found = true;
                        break;
                    }
                    const uint32_t itq = items[qq * cap + pick[qq]];
                    const int hq = qq >> 3;
                    const unsigned used2 = (used & ~item_banks(itq)) | item_banks(itc);
                    unsigned cls2[2] = {cls[0], cls[1]};
                    cls2[hq] &= ~(1u << (itq & 7u));
                    cls2[h] |= 1u << (itc & 7u);
                    const int alt = scan_best(qq, used2, cls2[hq]);
                    if (alt < 0) continue;
                    const uint32_t ita = items[qq * cap + alt];
                    account(qq, itq, -1);
                    account(p, itc, +1);
                    account(qq, ita, +1);
                    if (lane == 0) { pick[p] = base + src; pick[qq] = alt; }
                    used = used2 | item_banks(ita);
                    cls2[hq] |= 1u << (ita & 7u);
                    cls[0] = cls2[0]; cls[1] = cls2[1];
                    found = true;
                }
            }
            __syncwarp();
        }
        __syncwarp();
        // program words of the step
        const int pk = pick[my_pair];
        bool active = false;
        int row, k_mine = 0;
        if (pk >= 0) {
            const uint32_t it = items[my_pair * cap + pk];
            const unsigned kind = (it >> 20) & 3u;
            k_mine = int(it & 1023u);
            row = k_mine + 8;
            active = kind == 0u || kind == unsigned(1 + side);
        } else {
            row = __ffs(int(~cls[my_half] & 0xFFu)) - 1;     // an all-zero row of a class nobody in the half warp reads
        }
        const unsigned idle_mask = __ballot_sync(0xffffffffu, !active);
        const unsigned rowoff = unsigned(row) * 16u;
        uint32_t w;
        if (active) {
            const int s = sigma[qf[(size_t)(l_base + k_mine) * Cout + j]];
            w = uint32_t(2 * (s & 127)) | ((rowoff >> 8) << 8) | (uint32_t(1 + (s >> 7)) << 16) | ((rowoff & 255u) << 24);
        } else {
            const int nth = __popc(idle_mask & ((1u << lane) - 1u));
            const int zb = __fns(~used, 0, nth + 1);         // nth bank nobody looks up in this step
            w = uint32_t(4 * zb) | ((rowoff >> 8) << 8) | (1u << 14) | (3u << 16) | ((rowoff & 255u) << 24);
        }
        wq[step & 3] = w;
        if ((step & 3) == 3) prog[(size_t)(step >> 2) * 32 + lane] = make_uint4(wq[0], wq[1], wq[2], wq[3]);
        ++step;
        // retire the chosen items (the last item of the pair takes the freed place)
        __syncwarp();
        if (lane < 16 && pick[lane] >= 0) {
            const int last = cnt[lane] - 1;
            items[lane * cap + pick[lane]] = items[lane * cap + last];
            cnt[lane] = last;
        }
        total -= __popc(__ballot_sync(0xffffffffu, lane < 16 && pick[lane] >= 0));
        __syncwarp();
    }
    if (step & 3) {
        for (int e = step & 3; e < 4; ++e)
            wq[e] = uint32_t(4 * lane) | (1u << 14) | (3u << 16) | (uint32_t(((lane >> 1) & 7) * 16) << 24);
        prog[(size_t)(step >> 2) * 32 + lane] = make_uint4(wq[0], wq[1], wq[2], wq[3]);
    }
    if (lane == 0) {
        reinterpret_cast<int *>(plan + L.steps_off)[blockIdx.x] = (step + 3) >> 2;
        if (overflow) atomicOr(&hdr->fallback, 1);
    }
    block_done();
}

// ------------------------------------------------------------------------------------------------
// the convolution
// ------------------------------------------------------------------------------------------------
struct SchedParams {
    const unsigned char *plan;
    PlanLayout L;
    const float *input;
    float *output;
    int32_t *acc_out;
    int N, H, W, C, KH, KW, Cout;
    int sh, sw, dh, dw, ph, pw, OH, OW, K;
    long long M;              // end of the pixel range of this launch (all pixels: N*OH*OW)
    long long pix_base;       // first pixel of the range
    int g_base, g_count;      // channel groups [g_base, g_base + g_count) are served by this launch
    int split;                // consumer halves with barriers of their own (kernels with two or more slots)
    int dual;                 // plan_group_dual: lanes 16..31 repeat the channels of lanes 0..15 on a second pixel tile
    int tiles_n;              // channel tiles of 32*GW channels
    long long tiles_total;    // pixel tile groups x channel tiles
    int vec_ok;
    unsigned long long magic_c, magic_kw;   // ceil(2^40 / C), ceil(2^40 / KW): n / d == (n * magic) >> 40 for n*d < 2^40
    float in_floor;           // every input element is max(x, in_floor) as it is loaded: 0 = the producer's ReLU, -inf = none
};

__device__ __forceinline__ int fast_div(int n, unsigned long long magic)
{
    return int((static_cast<unsigned long long>(static_cast<unsigned>(n)) * magic) >> 40);
}

// Named barriers of dense_sched_kernel (barrier 0 is used once, after the table fill).
#define AXC_BAR(id, count) asm volatile("bar.sync %0, %1;" ::"n"(id), "n"(count) : "memory")
constexpr int kBarLoad = 1;   // loaders: pixel geometry of the tile group published
constexpr int kBarIter = 2;   // consumers + loaders: next activation buffers complete, current ones released
constexpr int kBarIterB = 3;  // the same for the second half of the pixel-tile slots (kernels with two or more slots)

// Tile group = NT pixel tiles of 16 pixels x (32*GW) channels, NT = (8/GW) * NTW.
// Warps 0..7  "consumers": warp w serves channel group w % GW and the NTW pixel tiles (w / GW)*NTW + i; it walks
//             the whole schedule of its (group, chunk) and reuses every program word for its NTW tiles.
// Warps 8..   "loaders" (LW of them, each owning whole pixel tiles): gather + quantise the activation rows of the
//             next (tile group, chunk) into the other set of buffers while the consumers work.  An activation
//             buffer is [8 zero rows + KC rows][16 pixel bytes]; the schedule guarantees that the two lanes of a
//             pair read the same row and that the 8 rows a half warp reads in one LDS.128 fall into 8 different
//             16-byte bank groups.
// The loaders also add up the raw taps of every pixel (the patch sums of the dequantisation).
template <int GW, int NTW, int LW>
__global__ void __launch_bounds__((kComputeWarps + LW) * 32, 1) dense_sched_kernel(const SchedParams P)
{
    constexpr int kLoaderWarps = LW;
    constexpr int kLoaderThreads = LW * 32;
    constexpr int kSchedThreads = (kComputeWarps + LW) * 32;
    constexpr int QS = 2;                            // a loader warp fetches 16 pixels x 2 neighbouring quads per load
    constexpr int SLOTS = kComputeWarps / GW;        // pixel-tile slots
    // With two or more slots the consumer warps form two halves (lower / upper slots) that meet the loaders at
    // barriers of their own, half an iteration apart: while one half dequantises and stores, waits or starts up,
    // the other keeps the shared-memory pipe busy.  The loaders fill the buffers of the lower half first.
    constexpr int kHalfCount = (kComputeWarps / 2 + LW) * 32;
    constexpr int kFullCount = (kComputeWarps + LW) * 32;
    const bool split = SLOTS >= 2 && P.split != 0;
    constexpr int NT = SLOTS * NTW;                  // pixel tiles per tile group
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const PlanHeader *hdr = reinterpret_cast<const PlanHeader *>(P.plan);
    if (hdr->fallback != 0) return;                  // the common-K kernel takes this call

    const unsigned dyn0 = (unsigned)__cvta_generic_to_shared(smem_raw);
    unsigned dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    const int KC = P.L.KC;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const DevQuant Q = *reinterpret_cast<const DevQuant *>(P.plan + kDevQuantOffset);
    const int nt_eff = P.dual ? 2 * NT : NT;         // pixel tiles per tile group
    // small tables below the table planes, then as many activation buffers as fit; the rest above the planes
    unsigned cur = (dyn0 + 15u) & ~15u;
    const unsigned sGeo = cur;               cur += unsigned(nt_eff) * kTilePix * 16u;
    const unsigned sAsum = cur;              cur += 3u * unsigned(nt_eff) * kTilePix * 4u;   // patch sums, 3 tile groups in rotation
    const bool tap_table = !P.vec_ok && P.K <= kTapTableMax;
    const unsigned sTap = cur;               cur += tap_table ? unsigned(P.K) * 8u : 0u;
    const int n_sched = P.L.G * P.L.NCH;
    const bool steps_in_smem = n_sched <= kStepsInSmemMax;
    const unsigned sSteps = cur;             cur += steps_in_smem ? unsigned(n_sched) * 4u : 0u;
    cur = (cur + 127u) & ~127u;
    const unsigned buf_bytes = unsigned(KC + 8) * 16u;
    const unsigned sBufA = cur;
    const int n_a = cur < kLutBase ? int((kLutBase - cur) / buf_bytes) : 0;
    const unsigned sBufB = kBuf1Base + 128u;         // after the 32 zero words
    const int n_b = int((kWindowEnd - sBufB) / buf_bytes);
    if (cur > kLutBase || n_a + n_b < 2 * nt_eff || dyn0 + dyn_size < kWindowEnd) {
        if (tid == 0) atomicExch(const_cast<int *>(&hdr->status), 2);
        return;
    }
    auto buf_addr = [&](int k) -> unsigned {          // k = parity * nt_eff + tile
        return k < n_a ? sBufA + unsigned(k) * buf_bytes : sBufB + unsigned(k - n_a) * buf_bytes;
    };

    // table image (already permuted and in plane layout), zero words, zero rows, small tables
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(P.plan + P.L.lut_off);
        for (int i = tid; i < 8192; i += kSchedThreads) sts128(kLutBase + unsigned(i) * 16u, __ldg(src + i));
        if (tid < 8) sts128(kBuf1Base + tid * 16, make_uint4(0, 0, 0, 0));
        for (int i = tid; i < 2 * nt_eff * 8; i += kSchedThreads) sts128(buf_addr(i >> 3) + unsigned(i & 7) * 16u, make_uint4(0, 0, 0, 0));
        if (steps_in_smem) {
            const int *sq = reinterpret_cast<const int *>(P.plan + P.L.steps_off);
            for (int i = tid; i < n_sched; i += kSchedThreads) sts32(sSteps + unsigned(i) * 4u, unsigned(__ldg(sq + i)));
        }
        if (tap_table) {
            for (int l = tid; l < P.K; l += kSchedThreads) {
                const int tap = l / P.C;
                const int cc = l - tap * P.C;
                const int ky = tap / P.KW;
                const int kx = tap - ky * P.KW;
                const int dy = ky * P.dh, dx = kx * P.dw;
                const int off = (dy * P.W + dx) * P.C + cc;     // fits: the table is only built for K <= 512
                sts32(sTap + unsigned(l) * 8u, unsigned(off));
                sts32(sTap + unsigned(l) * 8u + 4u, (unsigned(dy) & 0xFFFFu) | (unsigned(dx) << 16));
            }
        }
    }
    __syncthreads();

    const int NCH = P.L.NCH;
    const long long n_input = (long long)P.N * P.H * P.W * P.C;         // bounds of the debug flavour's checks
    const long long n_output = (long long)P.N * P.OH * P.OW * P.Cout;
    (void)n_input; (void)n_output;
    const long long my_groups = P.tiles_total > blockIdx.x ? (P.tiles_total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    // tile group number tl of this CTA -> first pixel and channel tile
    auto group_coords = [&](long long tl, long long *m0, int *nt) {
        const long long tile = blockIdx.x + tl * gridDim.x;
        const long long mt = tile / P.tiles_n;
        *nt = int(tile - mt * P.tiles_n);
        *m0 = P.pix_base + mt * (kTilePix * nt_eff);
    };

    if (warp >= kComputeWarps) {
        // ======================================== loaders ========================================
        const int ptid = tid - kComputeWarps * 32;          // 0..127
        const int p = ptid & 15;                            // this thread's pixel within every tile
        constexpr int kBatch = 2;                           // gathers in flight per thread (1 and 2 measure the same, 4 to 12 slower by 0.3 to 2 %)

        auto tap_value = [&](int l, int iy0, int ix0, long long base) -> float {
            unsigned off = 0, dd = 0;
            if (AXC_SHARED_OK(sTap + unsigned(l) * 8u, 8u, 0u, kWindowEnd, 107u))
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(off), "=r"(dd) : "r"(sTap + unsigned(l) * 8u));
            const unsigned iy = unsigned(iy0 + int(dd & 0xFFFFu)), ix = unsigned(ix0 + int(dd >> 16));
            return (iy < unsigned(P.H) && ix < unsigned(P.W) && AXC_GLOBAL_OK(base + int(off), n_input, 110u)) ? __ldg(P.input + base + int(off)) : 0.0f;
        };

        // half_sel: -1 all tiles, else only the tiles of that half of the slots; the pixel geometry of a tile group
        // is computed with its first part
        auto produce = [&](long long tl, int c, unsigned parity, int half_sel) {
            if (c == 0 && half_sel <= 0) {
                // geometry of the NT*16 pixels of the tile group: {element offset of the patch origin, iy0, ix0}
                long long m0; int nt;
                group_coords(tl, &m0, &nt);
                for (int x = ptid; x < nt_eff * kTilePix; x += kLoaderThreads) {
                    const long long pix = m0 + x;
                    int y0 = -(1 << 28), x0 = -(1 << 28);
                    long long b = 0;
                    if (pix < P.M) {
                        const int ow = int(pix % P.OW);
                        const long long t = pix / P.OW;
                        const int oh = int(t % P.OH);
                        const int n = int(t / P.OH);
                        y0 = oh * P.sh - P.ph;
                        x0 = ow * P.sw - P.pw;
                        b = (((long long)n * P.H + y0) * P.W + x0) * P.C;
                    }
                    if (AXC_SHARED_OK(sGeo + unsigned(x) * 16u, 16u, 0u, kWindowEnd, 108u)) {
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(sGeo + unsigned(x) * 16u), "r"(unsigned(b)), "r"(unsigned(b >> 32)) : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(sGeo + unsigned(x) * 16u + 8u), "r"(unsigned(y0)), "r"(unsigned(x0)) : "memory");
                    }
                }
                AXC_BAR(kBarLoad, kLoaderThreads);
            }
            const int l_base = c * KC;
            const int kc = min(KC, P.K - l_base);
            const int LQ = (kc + 3) >> 2;
            const int lq_first = (ptid & 31) >> 4;          // this thread's quads: lq_first + QS * s
            const int lw = ptid >> 5;                       // a loader warp owns whole tiles: lw, lw + LW, ...
            const int stages = (LQ + QS - 1) / QS;          // the same for both halves of the warp; quads >= LQ are masked
            for (int t = lw; t < nt_eff; t += kLoaderWarps) {
                if (half_sel >= 0 && (t >= nt_eff / 2 ? 1 : 0) != half_sel) continue;
                // Patch sum of pixel p (lanes 0..15): the raw taps added in K order, as the reference does
                // (tf2/src/approx_nn_conv_kernels.cpp:272-295).  Lane p holds the even quads of the pixel, lane
                // p + 16 the odd ones; the running sum takes the four values of the even quad, then the four of
                // the odd quad handed over by shuffles.  It is carried from chunk to chunk in shared memory.
                const unsigned sa = sAsum + ((unsigned(tl % 3) * unsigned(nt_eff) + unsigned(t)) * kTilePix + unsigned(p)) * 4u;
                float rs = 0.0f;
                if (c != 0 && (ptid & 31) < 16) rs = __uint_as_float(lds32(sa));
                const uint4 gq = lds128(sGeo + unsigned(t * kTilePix + p) * 16u);
                const long long base = (long long)(((unsigned long long)gq.y << 32) | gq.x);
                const int iy0 = int(gq.z), ix0 = int(gq.w);
                const unsigned bb = buf_addr(int(parity) * nt_eff + t) + 8u * 16u + unsigned(p);
                int l0 = l_base + lq_first * 4;
                int tap = l0 / P.C;
                int cc = l0 - tap * P.C;
                int ky = tap / P.KW;
                int kx = tap - ky * P.KW;
                for (int s0 = 0; s0 < stages; s0 += kBatch) {
                    float4 st[kBatch];
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (lq_first + QS * (s0 + u) < LQ) {
                            if (P.vec_ok) {
                                const int iy = iy0 + ky * P.dh, ix = ix0 + kx * P.dw;
                                if (iy >= 0 && iy < P.H && ix >= 0 && ix < P.W &&
                                    AXC_GLOBAL_OK(base + ((long long)(ky * P.dh) * P.W + kx * P.dw) * P.C + cc + 3, n_input, 111u))
                                    v = __ldg(reinterpret_cast<const float4 *>(
                                        P.input + base + ((long long)(ky * P.dh) * P.W + kx * P.dw) * P.C + cc));
                                cc += 4 * QS;
                                while (cc >= P.C) { cc -= P.C; if (++kx >= P.KW) { kx = 0; ++ky; } }
                            } else {
                                float e4[4] = {0.f, 0.f, 0.f, 0.f};
                                if (tap_table) {
#pragma unroll
                                    for (int e = 0; e < 4; ++e)
                                        if (l0 + e < P.K) e4[e] = tap_value(l0 + e, iy0, ix0, base);
                                } else {
                                    int tp = fast_div(l0, P.magic_c);
                                    int c2 = l0 - tp * P.C;
                                    int y2 = fast_div(tp, P.magic_kw);
                                    int x2 = tp - y2 * P.KW;
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        if (l0 + e < P.K) {
                                            const int iy = iy0 + y2 * P.dh, ix = ix0 + x2 * P.dw;
                                            if (iy >= 0 && iy < P.H && ix >= 0 && ix < P.W &&
                                                AXC_GLOBAL_OK(base + ((long long)(y2 * P.dh) * P.W + x2 * P.dw) * P.C + c2, n_input, 112u))
                                                e4[e] = __ldg(P.input + base + ((long long)(y2 * P.dh) * P.W + x2 * P.dw) * P.C + c2);
                                        }
                                        if (++c2 >= P.C) { c2 = 0; if (++x2 >= P.KW) { x2 = 0; ++y2; } }
                                    }
                                }
                                v = make_float4(e4[0], e4[1], e4[2], e4[3]);
                            }
                            l0 += 4 * QS;
                        }
                        // the producer's ReLU, applied to the raw taps (quantiser and patch sum both see max(x, 0))
                        v.x = max_keep_nan(v.x, P.in_floor); v.y = max_keep_nan(v.y, P.in_floor);
                        v.z = max_keep_nan(v.z, P.in_floor); v.w = max_keep_nan(v.w, P.in_floor);
                        st[u] = v;
                    }
                    // quantise -> rows of the activation buffer; lanes = pixels, so the byte stores of a warp fall
                    // into two groups of four consecutive words
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        if (s0 + u < stages) {                  // uniform over the warp
                            const int lq = lq_first + QS * (s0 + u);
                            const unsigned a = bb + unsigned(lq * 4) * 16u;
                            const float4 v = st[u];             // zeros beyond the chunk
                            if (lq < LQ) {
                                sts8(a, q_u8(v.x, Q.in_off, Q.in_inv));
                                if (lq * 4 + 1 < kc) sts8(a + 16, q_u8(v.y, Q.in_off, Q.in_inv));
                                if (lq * 4 + 2 < kc) sts8(a + 32, q_u8(v.z, Q.in_off, Q.in_inv));
                                if (lq * 4 + 3 < kc) sts8(a + 48, q_u8(v.w, Q.in_off, Q.in_inv));
                            }
                            const float ox = __shfl_down_sync(0xffffffffu, v.x, 16), oy = __shfl_down_sync(0xffffffffu, v.y, 16);
                            const float oz = __shfl_down_sync(0xffffffffu, v.z, 16), ow = __shfl_down_sync(0xffffffffu, v.w, 16);
                            rs = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(rs, v.x), v.y), v.z), v.w);
                            rs = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(rs, ox), oy), oz), ow);
                        }
                    }
                }
                if ((ptid & 31) < 16) sts32(sa, __float_as_uint(rs));
            }
        };

        long long tl = 0;
        int c = 0;
        unsigned parity = 0;
        const long long total_iters = my_groups * NCH;
        if (split) {
            if (my_groups > 0) produce(0, 0, 0u, 0);
            AXC_BAR(kBarIter, kHalfCount);
            if (my_groups > 0) produce(0, 0, 0u, 1);
            AXC_BAR(kBarIterB, kHalfCount);
            for (long long it = 0; it < total_iters; ++it) {
                if (++c == NCH) { c = 0; ++tl; }
                parity ^= 1u;
                if (it + 1 < total_iters) produce(tl, c, parity, 0);
                AXC_BAR(kBarIter, kHalfCount);
                if (it + 1 < total_iters) produce(tl, c, parity, 1);
                AXC_BAR(kBarIterB, kHalfCount);
            }
        } else {
            if (my_groups > 0) produce(0, 0, 0u, -1);
            AXC_BAR(kBarIter, kFullCount);
            for (long long it = 0; it < total_iters; ++it) {
                if (++c == NCH) { c = 0; ++tl; }
                parity ^= 1u;
                if (it + 1 < total_iters) produce(tl, c, parity, -1);
                AXC_BAR(kBarIter, kFullCount);
            }
        }
        return;
    }

    // ========================================= consumers =========================================
    const int gl = warp % GW, slot = warp / GW;
    const int half = P.dual ? (lane >> 4) : 0;       // which of the warp's two pixel tiles this lane works on
    const int chan_lane = P.dual ? (lane & 15) : lane;
    const int *steps_q = reinterpret_cast<const int *>(P.plan + P.L.steps_off);
    const uint4 *prog = reinterpret_cast<const uint4 *>(P.plan + P.L.prog_off);
    const float *bsum = reinterpret_cast<const float *>(P.plan + P.L.bsum_off);
    int acc[NTW][kTilePix];
    unsigned base0[NTW], base1[NTW];               // this warp's activation buffers, parity 0 / 1
#pragma unroll
    for (int i = 0; i < NTW; ++i) {
#pragma unroll
        for (int x = 0; x < kTilePix; ++x) acc[i][x] = 0;
        const int tile = P.dual ? 2 * (slot * NTW + i) + half : slot * NTW + i;
        base0[i] = buf_addr(tile);
        base1[i] = buf_addr(nt_eff + tile);
    }

    // the schedule of (channel tile nt, chunk c) that this warp walks
    auto sched_of = [&](int nt, int c, const uint4 **pp, int *nq) {
        const int gi = nt * GW + gl;
        *nq = 0;
        *pp = prog;
        if (gi < P.g_count) {
            const int sc = (P.g_base + gi) * NCH + c;
            const int stored = steps_in_smem ? int(lds32(sSteps + unsigned(sc) * 4u)) : __ldg(steps_q + sc);
            *nq = min(max(stored, 0), P.L.sqcap);          // never walk beyond the block's reserve
            *pp = prog + (size_t)sc * P.L.sqcap * 32 + lane;
        }
    };

    const uint4 *pp = prog;
    int nq = 0;
    uint4 w_a = make_uint4(0, 0, 0, 0), w_b = make_uint4(0, 0, 0, 0);   // two quads of look-ahead
    long long m0 = 0;
    int nt = 0;
    if (my_groups > 0) {
        group_coords(0, &m0, &nt);
        sched_of(nt, 0, &pp, &nq);
        if (nq > 0) w_a = __ldg(pp);
        if (nq > 1) w_b = __ldg(pp + 32);
    }
    const bool upper_half = slot >= SLOTS / 2;
    auto iter_barrier = [&]() {
        if (!split) AXC_BAR(kBarIter, kFullCount);
        else if (upper_half) AXC_BAR(kBarIterB, kHalfCount);
        else AXC_BAR(kBarIter, kHalfCount);
    };
    iter_barrier();

    unsigned parity = 0;
    float t2 = 0.0f;          // m1 * bSum[j] of this lane's channel
    int t2_nt = -1;
    for (long long tl = 0; tl < my_groups; ++tl) {
        long long m0_next = 0;
        int nt_next = 0;
        if (tl + 1 < my_groups) group_coords(tl + 1, &m0_next, &nt_next);
        {
            const int j = (P.g_base + nt * GW + gl) * 32 + chan_lane;
            if (nt != t2_nt) { t2 = j < P.Cout ? __fmul_rn(Q.m1, __ldg(bsum + j)) : 0.0f; t2_nt = nt; }
        }
        for (int c = 0; c < NCH; ++c) {
            // first two quads of the next (tile group, chunk): requested now, consumed after the barrier
            const uint4 *pp_n = prog;
            int nq_n = 0;
            uint4 n_a = make_uint4(0, 0, 0, 0), n_b = make_uint4(0, 0, 0, 0);
            if (c + 1 < NCH) sched_of(nt, c + 1, &pp_n, &nq_n);
            else if (tl + 1 < my_groups) sched_of(nt_next, 0, &pp_n, &nq_n);
            if (nq_n > 0) n_a = __ldg(pp_n);
            if (nq_n > 1) n_b = __ldg(pp_n + 32);

            for (int q = 0; q < nq; ++q) {
                const uint4 wq = w_a;
                w_a = w_b;
                if (q + 2 < nq) w_b = __ldg(pp + (size_t)(q + 2) * 32);
                const uint32_t ws[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t w = ws[e];
                    const unsigned rowoff = (w >> 24) | (w & 0x3F00u);     // 16 * activation row
                    // byte selectors {column byte of w, activation byte i, plane byte of w, 0}; an idle lane (bit 14)
                    // takes 0 for the activation byte, whatever row it reads along with its neighbour
                    const unsigned idle = (w >> 14) & 1u;
                    const unsigned sel0 = 0xA240u + idle * 0x60u, sel_inc = 16u - idle * 16u;
                    const unsigned sel1 = sel0 + sel_inc, sel2 = sel1 + sel_inc, sel3 = sel2 + sel_inc;
#pragma unroll
                    for (int i = 0; i < NTW; ++i) {
                        const uint4 av = lds128((parity ? base1[i] : base0[i]) + rowoff);
                        const unsigned aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                        for (int i4 = 0; i4 < kTilePix / 4; ++i4) {
                            // table address = {column byte of w, activation byte, plane byte of w, 0}
                            acc[i][i4 * 4 + 0] += int(lds16(prmt_r(w, aw[i4], sel0)));
                            acc[i][i4 * 4 + 1] += int(lds16(prmt_r(w, aw[i4], sel1)));
                            acc[i][i4 * 4 + 2] += int(lds16(prmt_r(w, aw[i4], sel2)));
                            acc[i][i4 * 4 + 3] += int(lds16(prmt_r(w, aw[i4], sel3)));
                        }
                    }
                }
            }
            pp = pp_n; nq = nq_n; w_a = n_a; w_b = n_b;
            iter_barrier();
            parity ^= 1u;
        }
        // ---- the tile group is complete: dequantise and store ------------------------------------
        {
            const int j = (P.g_base + nt * GW + gl) * 32 + chan_lane;
            const bool live = (nt * GW + gl) < P.g_count && j < P.Cout;
#pragma unroll
            for (int i = 0; i < NTW; ++i) {
                const int tile = P.dual ? 2 * (slot * NTW + i) + half : slot * NTW + i;
#pragma unroll
                for (int x = 0; x < kTilePix; ++x) {
                    const long long pix = m0 + tile * kTilePix + x;
                    const float a_sum = __uint_as_float(lds32(sAsum + ((unsigned(tl % 3) * unsigned(nt_eff) + unsigned(tile)) * kTilePix + unsigned(x)) * 4u));
                    if (live && pix < P.M && AXC_GLOBAL_OK(pix * P.Cout + j, n_output, 113u)) {
                        const float t0 = __fmul_rn(float(acc[i][x]), Q.s1s2);
                        const float t1 = __fmul_rn(Q.m2, a_sum);
                        P.output[pix * P.Cout + j] = __fsub_rn(__fadd_rn(__fadd_rn(t0, t1), t2), Q.km1m2);
                        asm volatile("" ::: "memory");      // the tap may be the same memory (integer sums only): keep the order
                        if (P.acc_out) P.acc_out[pix * P.Cout + j] = acc[i][x];
                    }
                    acc[i][x] = 0;
                }
            }
        }
        m0 = m0_next;
        nt = nt_next;
    }
}

template <int GW, int NTW, int LW>
int launch_sched_variant(SchedParams P, const DeviceInfo &di, cudaStream_t stream)
{
    constexpr int kSchedThreads = (kComputeWarps + LW) * 32;
    constexpr int NT = (kComputeWarps / GW) * NTW;
    const int nt_eff = P.dual ? 2 * NT : NT;
    P.tiles_n = (P.g_count + GW - 1) / GW;
    P.tiles_total = ((P.M - P.pix_base + kTilePix * nt_eff - 1) / (kTilePix * nt_eff)) * P.tiles_n;
    AXC_CUDA(cudaFuncSetAttribute(dense_sched_kernel<GW, NTW, LW>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
    const long long grid = P.tiles_total < di.sm_count ? P.tiles_total : di.sm_count;
    dense_sched_kernel<GW, NTW, LW><<<unsigned(grid), kSchedThreads, size_t(di.max_smem_optin), stream>>>(P);
    AXC_CUDA(cudaGetLastError());
    count_launch();
    return AXC_OK;
}

// Activation buffers that fit beside the table (the kernel repeats this computation with the real window base).
int buffers_that_fit(const SchedParams &P, int NT, unsigned smem_base)
{
    unsigned cur = (smem_base + 15u) & ~15u;                  // first dynamic byte of the window, as probed on this device
    cur += unsigned(NT) * kTilePix * 16u;
    cur += 3u * unsigned(NT) * kTilePix * 4u;
    if (!P.vec_ok && P.K <= kTapTableMax) cur += unsigned(P.K) * 8u;
    if (P.L.G * P.L.NCH <= kStepsInSmemMax) cur += unsigned(P.L.G * P.L.NCH) * 4u;
    cur = (cur + 127u) & ~127u;
    const unsigned buf_bytes = unsigned(P.L.KC + 8) * 16u;
    const int n_a = cur < kLutBase ? int((kLutBase - cur) / buf_bytes) : 0;
    const int n_b = int((kWindowEnd - (kBuf1Base + 128u)) / buf_bytes);
    return n_a + n_b;
}

}  // namespace

// Next run of channel groups for a launch: `rem` groups are left; returns the GW of the launch and how many
// groups it covers.  Whole multiples of 8 go together; 5 and 6 are cut into 4 + 1 and 4 + 2; 3 and 7 are rounded
// up to a launch of 4 resp. 8 with one idle consumer-warp column (cheaper than a second launch).
static void next_group_run(int rem, int K, int *gw, int *count)
{
    if (rem >= 8) { *gw = 8; *count = (rem / 8) * 8; return; }
    if (rem == 7) { *gw = 8; *count = 7; return; }
    if (rem >= 4) { *gw = 4; *count = 4; return; }
    if (rem == 3 && K <= 64) { *gw = 2; *count = 2; return; }   // short schedules: 2 + 1 measured faster than 4 with a gap
    if (rem == 3) { *gw = 4; *count = 3; return; }
    *gw = rem; *count = rem;
}

PlanLayout plan_layout(int K, int Cout)
{
    PlanLayout L;
    L.G = (Cout + 31) / 32;
    // Chunk length: two sets of activation buffers of (KC + 8) * 16 bytes must fit beside the table for every
    // pixel-tile slot of the kernel.  The groups are served in runs of 8, 4, 2 and 1 (launch_dense_sched); the
    // smallest run decides: 8 slots for a run of one group, 4 for two, 2 for four, 1 for eight.
    int smallest = 8;
    for (int rem = L.G; rem > 0;) {
        int gw, count;
        next_group_run(rem, K, &gw, &count);
        if (gw < smallest) smallest = gw;
        rem -= count;
    }
    // a group of at most 16 channels launched alone runs two pixel tiles per warp: twice the buffers
    const int kc_max = plan_group_dual(L.G - 1, L.G, Cout, K) ? 152 : smallest == 1 ? 160 : smallest == 2 ? 304 : kMaxChunk;
    L.NCH = (K + kc_max - 1) / kc_max;
    L.KC = (((K + L.NCH - 1) / L.NCH) + 3) & ~3;
    if (L.KC > kc_max) L.KC = kc_max;
    L.sqcap = (2 * L.KC + 3) / 4 + 1;               // room for twice the ideal number of steps
    auto r256 = [](size_t v) { return (v + 255) & ~size_t(255); };
    size_t off = 256;
    L.qf_off = off;      off += r256(size_t(K) * Cout);
    L.sigma_off = off;   off += 256;
    L.lut_off = off;     off += 131072;
    L.bsum_off = off;    off += r256(size_t(Cout) * 4);
    L.steps_off = off;   off += r256(size_t(L.G) * L.NCH * 4);
    L.prog_off = off;    off += size_t(L.G) * L.NCH * L.sqcap * 512;
    L.total = off;
    return L;
}

static DevQuant host_dev_quant(const Quant &q, int K)
{
    DevQuant d;
    d.in_off = q.in_off; d.in_inv = q.in_inv; d.f_off = q.f_off; d.f_inv = q.f_inv;
    d.s1s2 = q.s1s2; d.m1 = q.m1; d.m2 = q.m2;
    volatile float kf = float(K);
    volatile float t3 = kf * q.m1m2;
    d.km1m2 = t3;
    return d;
}

__global__ void quant_store_kernel(DevQuant host_q, const float *__restrict__ ranges, int K, DevQuant *out)
{
    *out = ranges ? dev_quant_from_ranges(ranges, K) : host_q;
}

// For calls that do not go through launch_plan (common-K kernel only).
int launch_quant(const Quant &q, const float *ranges_dev, int K, unsigned char *plan, cudaStream_t stream)
{
    quant_store_kernel<<<1, 1, 0, stream>>>(host_dev_quant(q, K), ranges_dev, K, reinterpret_cast<DevQuant *>(plan + kDevQuantOffset));
    AXC_CUDA(cudaGetLastError());
    count_launch();
    return AXC_OK;
}

int launch_plan(const uint16_t *lut_dev, unsigned table_uid, const Geom &g, const Quant &q, const float *ranges_dev,
                const float *filter, unsigned char *plan, const PlanLayout &L, uint8_t *qf_debug, cudaStream_t stream)
{
    PlanHeader want = {};
    want.magic = kPlanMagic;
    want.K = g.K; want.Cout = g.Cout; want.G = L.G; want.NCH = L.NCH; want.KC = L.KC; want.sqcap = L.sqcap;
    want.table_uid = table_uid;
    PlanHeader *hdr = reinterpret_cast<PlanHeader *>(plan);
    AXC_CUDA(cudaMemsetAsync(&hdr->dirty, 0, sizeof(int), stream));
    const long long count = (long long)g.K * g.Cout;
    const DevQuant *dq = reinterpret_cast<const DevQuant *>(plan + kDevQuantOffset);
    plan_check_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(filter, count, host_dev_quant(q, g.K), ranges_dev, g.K, plan, L,
                                                                         qf_debug, want);
    AXC_CUDA(cudaGetLastError());
    {
        // the local search of plan_sigma_kernel needs 640 bytes of shared memory per schedule block
        const int blocks = L.G * L.NCH;
        const int search_blocks = blocks <= kSigmaMaxBlocks ? blocks : 0;
        const size_t sigma_smem = size_t(search_blocks) * (128 + 32 + 4) * sizeof(int);
        AXC_CUDA(cudaFuncSetAttribute(plan_sigma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSigmaMaxBlocks * 164 * sizeof(int))));
        plan_sigma_kernel<<<1, 256, sigma_smem, stream>>>(plan + L.qf_off, g.K, g.Cout, L, search_blocks, plan + L.sigma_off, hdr, want, dq);
        AXC_CUDA(cudaGetLastError());
    }
    const unsigned blocks = unsigned(L.G * L.NCH + 256 + (g.Cout + 31) / 32);
    const size_t sched_smem = size_t(16) * 2 * L.KC * sizeof(uint32_t);   // the items of the 16 lane pairs
    AXC_CUDA(cudaFuncSetAttribute(plan_build_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sched_smem)));
    plan_build_kernel<<<blocks, 32, sched_smem, stream>>>(filter, lut_dev, plan, L, g.K, g.Cout);
    AXC_CUDA(cudaGetLastError());
    count_launch(3);
    return AXC_OK;
}

int launch_dense_sched(const Geom &g, const float *input, float *output,
                       const unsigned char *plan, const PlanLayout &L, int32_t *acc_out, const DeviceInfo &di,
                       cudaStream_t stream)
{
    SchedParams P;
    P.plan = plan; P.L = L; P.input = input; P.output = output; P.acc_out = acc_out;
    P.N = g.N; P.H = g.H; P.W = g.W; P.C = g.C; P.KH = g.KH; P.KW = g.KW; P.Cout = g.Cout;
    P.sh = g.sh; P.sw = g.sw; P.dh = g.dh; P.dw = g.dw; P.ph = g.ph; P.pw = g.pw; P.OH = g.OH; P.OW = g.OW;
    P.K = g.K; P.M = g.M; P.pix_base = 0; P.tiles_n = 0; P.tiles_total = 0;
    P.vec_ok = (g.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(input) & 15u) == 0);
    P.dual = 0;
    P.in_floor = g.ep.input_relu ? 0.0f : -INFINITY;
    // n / d == (n * magic) >> 40 holds while n * d < 2^40; launch_dense keeps shapes beyond that on the common-K kernel
    P.magic_c = ((1ull << 40) + unsigned(g.C) - 1) / unsigned(g.C);
    P.magic_kw = ((1ull << 40) + unsigned(g.KW) - 1) / unsigned(g.KW);
    // The 8 consumer warps of a CTA serve GW channel groups x 8/GW pixel-tile slots, GW a power of two.  A
    // group count that is not one is cut into runs (next_group_run), one launch each, so that few consumer warps
    // are left without a group.
    int g_done = 0;
    while (g_done < L.G) {
        int gw, count;
        next_group_run(L.G - g_done, g.K, &gw, &count);
        P.g_base = g_done;
        P.g_count = count;
        P.dual = (count == 1 && plan_group_dual(g_done, L.G, g.Cout, g.K)) ? 1 : 0;
        // two consumer halves pay off once an iteration is long enough to hide the second barrier (measured:
        // +1-4 % for K >= 64, -14 % for K = 32)
        P.split = L.KC >= 64 ? 1 : 0;
        // pixel tiles per consumer warp: as many as the shared-memory budget allows (two sets of buffers)
        const int slots = (kComputeWarps / gw) * (P.dual ? 2 : 1);   // pixel tiles in flight per unit of NTW
        int ntw = 4;
        while (ntw > 1 && buffers_that_fit(P, slots * ntw, di.smem_base) < 2 * slots * ntw) ntw >>= 1;
        if (buffers_that_fit(P, slots * ntw, di.smem_base) < 2 * slots * ntw) return AXC_INTERNAL;
        // Tile groups are handed out round-robin to one CTA per SM, so a launch takes ceil(groups / SMs) rounds.
        // Choose between one launch (any admissible number of tiles per warp) and a main launch of whole rounds
        // followed by a tail launch with smaller tile groups for the pixels that are left; estimate: a round
        // costs per warp step 18 shared-memory cycles per tile plus about 2.6 that do not depend on the tiles.
        const long long unit = (long long)kTilePix * slots;           // pixels per tile group and unit of NTW
        const int tiles_n = (count + gw - 1) / gw;
        const double step_us = double(g.K) * 1.08 * 8.0 / 1965.0;     // one pipe cycle per step, in microseconds
        auto rounds = [&](long long pixels, int n) -> long long {
            const long long groups = (pixels + unit * n - 1) / (unit * n) * tiles_n;
            return (groups + di.sm_count - 1) / di.sm_count;
        };
        auto cost = [&](long long pixels, int n) -> double {
            return pixels > 0 ? double(rounds(pixels, n)) * (18.0 * n + 2.6) * step_us + 12.0 : 0.0;   // + launch, table fill
        };
        int best_main = ntw, best_tail = 0;
        long long best_split = g.M;
        double best_cost = 1e300;
        for (int n = ntw; n >= 1; n >>= 1) {
            const double c1 = cost(g.M, n);
            if (c1 < best_cost) { best_cost = c1; best_main = n; best_tail = 0; best_split = g.M; }
            // main launch: the whole rounds of the pixel groups; tail: the rest
            const long long pg = (g.M + unit * n - 1) / (unit * n);
            const long long full_groups = (pg * tiles_n / di.sm_count) * di.sm_count;
            const long long pg_main = full_groups / tiles_n;
            if (pg_main <= 0 || pg_main >= pg) continue;
            const long long split = pg_main * unit * n;
            for (int nt2 = n; nt2 >= 1; nt2 >>= 1) {
                const double c2 = cost(split, n) + cost(g.M - split, nt2);
                if (c2 < best_cost) { best_cost = c2; best_main = n; best_tail = nt2; best_split = split; }
            }
        }
        int rc = AXC_INTERNAL;
#define AXC_DISPATCH(GWV, NTWV)                                                       \
        if (gw == GWV) {                                                              \
            if (NTWV == 4) rc = launch_sched_variant<GWV, 4, 4>(P, di, stream);       \
            else if (GWV == 1 && NTWV == 2) rc = launch_sched_variant<1, 2, 8>(P, di, stream);  \
            else if (GWV == 1) rc = launch_sched_variant<1, 1, 8>(P, di, stream);     \
            else if (NTWV == 2) rc = launch_sched_variant<GWV, 2, 4>(P, di, stream);  \
            else rc = launch_sched_variant<GWV, 1, 4>(P, di, stream);                 \
        }
        P.pix_base = 0; P.M = best_split;
        AXC_DISPATCH(1, best_main)
        AXC_DISPATCH(2, best_main)
        AXC_DISPATCH(4, best_main)
        AXC_DISPATCH(8, best_main)
        if (rc) return rc;
        if (best_tail > 0) {
            P.pix_base = best_split; P.M = g.M;
            rc = AXC_INTERNAL;
            AXC_DISPATCH(1, best_tail)
            AXC_DISPATCH(2, best_tail)
            AXC_DISPATCH(4, best_tail)
            AXC_DISPATCH(8, best_tail)
        }
#undef AXC_DISPATCH
        if (rc) return rc;
        g_done += count;
    }
    return AXC_OK;
}

AXC_DEFINE_BOUNDS_READER(bounds_record_sched)

int plan_info(const void *workspace, int32_t out4[4], cudaStream_t stream)
{
    AXC_CUDA(cudaStreamSynchronize(stream));
    PlanHeader h;
    AXC_CUDA(cudaMemcpy(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost));
    out4[0] = h.dirty; out4[1] = h.fallback; out4[2] = h.status; out4[3] = 0;
    if (h.magic == kPlanMagic && h.G > 0 && h.NCH > 0 && h.G * h.NCH <= 65536) {
        const PlanLayout L = plan_layout(h.K, h.Cout);
        std::vector<int> steps(size_t(h.G) * h.NCH);
        AXC_CUDA(cudaMemcpy(steps.data(), static_cast<const unsigned char *>(workspace) + L.steps_off,
                            steps.size() * sizeof(int), cudaMemcpyDeviceToHost));
        long long quads = 0;
        for (int v : steps) quads += v;
        const long long ideal = (long long)h.G * ((h.K + 3) / 4);
        out4[3] = ideal > 0 ? int(quads * 1000 / ideal) : 0;
    }
    return AXC_OK;
}

}  // namespace axc
