// Plan (per-filter schedule) kept in the caller's workspace for the bank-scheduled dense kernel.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

namespace axc {

struct Geom;
struct Quant;
struct DeviceInfo;

// K elements per schedule chunk: a program word addresses activation rows 0..1023 (8 zero rows + the chunk).
constexpr int kMaxChunk = 1016;

struct PlanHeader {
    uint32_t magic;
    int K, Cout, G, NCH, KC, sqcap;
    uint32_t table_uid;
    uint32_t f_off_bits, f_inv_bits;
    int dirty;      // set by plan_check when the stored plan does not belong to this filter / table
    int fallback;   // set when a schedule did not fit: the common-K kernel serves the call
    int status;     // 0 fine; 2 shared-memory layout check failed
    int blocks_done;   // plan_build blocks that have finished: the last one writes `magic`
    int pad[2];
};

// Quantisation parameters of a call as the kernels read them.  Filled from host values, or on the device from
// four range scalars that live in device memory (no host round trip).  Kept in the workspace header.
struct DevQuant {
    float in_off, in_inv, f_off, f_inv, s1s2, m1, m2, km1m2;
};
constexpr size_t kDevQuantOffset = 128;   // inside the 256-byte plan header block

struct PlanLayout {
    int G, NCH, KC, sqcap;   // channel groups of 32, K chunks, chunk length, step-quads reserved per (group, chunk)
    size_t qf_off, sigma_off, lut_off, bsum_off, steps_off, prog_off, total;
};

PlanLayout plan_layout(int K, int Cout);

// A channel group with at most 16 live channels that is served by a launch of its own (the last group when the
// group count is 1, 5, 9, ...: see next_group_run) runs "dual": lanes 16..31 repeat the channels of lanes 0..15
// on a second pixel tile, so no lane is left without work.
// Doubling the pixel tiles caps the K chunk at 152 for the whole filter, so with several groups it is only done
// when K fits one such chunk anyway.
__host__ __device__ inline bool plan_group_dual(int g, int G, int Cout, int K)
{
    return g == G - 1 && (G % 4) == 1 && Cout - 32 * g <= 16 && (G == 1 || K <= 152);
}

// Writes the DevQuant block of `plan`: from the host values `q`, or - when ranges_dev is given - on the device
// from {in_min, in_max, f_min, f_max} read there (same arithmetic as the host: tf2/src/approx_ops_types.h:29-49,135-197).
// launch_plan does the same as part of its first kernel; launch_quant is for calls that skip the plan.
int launch_quant(const Quant &q, const float *ranges_dev, int K, unsigned char *plan, cudaStream_t stream);

int launch_plan(const uint16_t *lut_dev, unsigned table_uid, const Geom &g, const Quant &q, const float *ranges_dev,
                const float *filter, unsigned char *plan, const PlanLayout &L, uint8_t *qf_debug, cudaStream_t stream);

int launch_dense_sched(const Geom &g, const float *input, float *output,
                       const unsigned char *plan, const PlanLayout &L, int32_t *acc_out, const DeviceInfo &di,
                       cudaStream_t stream);

// Header fields of the plan in `workspace` (diagnostics; synchronises the stream).
int plan_info(const void *workspace, int32_t out4[4], cudaStream_t stream);

}  // namespace axc
