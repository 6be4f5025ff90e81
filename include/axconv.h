/*
 * axconv - table-driven approximate convolution for NVIDIA B200 (sm_100a).
 *
 * C ABI of the forward pass of TFApprox's `ApproxConv2DWithMinMaxVars` op and of a
 * depthwise variant.  Every 8-bit x 8-bit product of the convolution is a lookup in a
 * 256x256 uint16 truth table, index (activation << 8) | weight.
 *
 * The reference (ehw-fit/tf-approximate, tf2 generation) has no C ABI: its boundary is
 * the TensorFlow op kernel `ApproxConv2DOp::Compute` (tf2/src/approx_nn_conv_ops.cpp:420-460).
 * Each entry point below names the part of that op it stands in for, so that an op-kernel
 * shim can keep the op registration (tf2/src/approx_nn_ops.cpp:38-54) byte for byte and
 * forward to this library.
 *
 * Conventions: plain pointers and sizes only; every function returns an axc_status
 * (0 = OK) and never aborts; tensor pointers are DEVICE pointers on `device` unless a
 * parameter says otherwise; launches are asynchronous on `stream` (a cudaStream_t passed
 * as void*, NULL = the legacy default stream).  Calls on different streams or devices may
 * run concurrently from different host threads.
 */
#ifndef AXCONV_H
#define AXCONV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  The numeric values of the first three are TensorFlow's error codes for
 * the conditions the reference reports through OP_REQUIRES
 * (tf2/src/approx_nn_conv_ops.cpp:120-121,160-163,224-232,274-303,315-341,521;
 *  tf2/src/approx_ops_types.h:213). */
typedef enum {
    AXC_OK = 0,
    AXC_INVALID_ARGUMENT = 3,  /* bad shapes/strides/dilations/num_bits, unreadable table  */
    AXC_UNIMPLEMENTED = 12,    /* EXPLICIT padding, NCHW, grouped (non-depthwise) shapes   */
    AXC_INTERNAL = 13,         /* e.g. workspace missing or too small                      */
    AXC_CUDA_ERROR = 100       /* a CUDA call failed; see axc_last_cuda_error()            */
} axc_status;

enum { AXC_PADDING_SAME = 0, AXC_PADDING_VALID = 1, AXC_PADDING_EXPLICIT = 2 };
enum { AXC_FORMAT_NHWC = 0, AXC_FORMAT_NCHW = 1 };
/* How the looked-up products of one output are added up.
 * AXC_ACCUM_EXACT_I32 (default): exact integer sum, any order; the fp32 output is the dequantisation of the
 *   exact sum.  Equal to the reference bit for bit whenever the reference's own running total is exact.
 * AXC_ACCUM_REFERENCE_F32: the reference's arithmetic, `total += float(entry)` in K order with an fp32 running
 *   total (tf2/src/approx_nn_conv_kernels.cpp:245-246), which rounds once a partial sum passes 2^24.  Output
 *   bits equal the reference's CPU kernel for every K.  Where the table and K prove that no partial sum can
 *   round (K * largest entry <= 2^24 * the power of two dividing every entry) the fast integer kernel serves
 *   the call, since both give the same bits; otherwise a kernel that walks K in order does (about half the
 *   speed).  Depthwise calls ignore the field (K = kh*kw never rounds). */
enum { AXC_ACCUM_EXACT_I32 = 0, AXC_ACCUM_REFERENCE_F32 = 1 };
/* Whether the dense op prepares a per-filter lookup plan (kept in the workspace, built in 3-90 ms, reused while the
 * filter is unchanged) or serves the call without one.
 * AXC_PLAN_KEEP (default): inference - the plan makes every table lookup conflict-free (about 1.8 x the speed).
 * AXC_PLAN_NONE: filters that change from call to call (training steps): the kernel that walks K in order serves
 *   the call, nothing is prepared and nothing has to be rebuilt.  Same results bit for bit. */
enum { AXC_PLAN_KEEP = 0, AXC_PLAN_NONE = 1 };

/* Geometry of one call: what ApproxConv2DParameters + ApproxConv2DDimensions carry
 * (tf2/src/approx_nn_conv_ops.h:36-98, filled at tf2/src/approx_nn_conv_ops.cpp:254-404).
 * input  [n,h,w,c] fp32 NHWC; filter [kh,kw,filter_c,cout] fp32 (HWIO).
 * For axc_conv2d_forward filter_c must equal c.  For the depthwise entry point filter_c
 * must equal c and `cout` is the channel multiplier. */
typedef struct {
    int32_t n, h, w, c;
    int32_t kh, kw, filter_c, cout;
    int32_t stride_h, stride_w;
    int32_t dil_h, dil_w;
    int32_t padding;      /* AXC_PADDING_*  */
    int32_t data_format;  /* AXC_FORMAT_*   */
    int32_t accumulate;   /* AXC_ACCUM_*: 0 = exact int32 sum (default), 1 = the reference's fp32 running total */
    int32_t plan;         /* AXC_PLAN_*: 0 = keep a lookup plan per filter (default), 1 = none (changing filters) */
} axc_conv_desc;

/* Optional taps into the integer pipeline, for parity checks (device pointers, any may be
 * NULL).  No counterpart in the reference, whose integer operands live only in its
 * temporary im2col buffer (tf2/src/approx_nn_conv_ops.cpp:126-153). */
typedef struct {
    uint8_t *qinput;  /* [n,h,w,c]            element-wise quantised input               */
    uint8_t *qfilter; /* [kh*kw*filter_c,cout] element-wise quantised filter             */
    int32_t *acc;     /* output shape          exact integer sum of the looked-up entries; when the call is
                                               served in reference order: that fp32 running total as an integer */
} axc_debug_out;

typedef struct axc_table axc_table;

/* ---- truth table: BaseTableApproxOpType_t (tf2/src/approx_ops_types.h:99-122,205-216)
 *      and its device copy (tf2/src/cuda/approx_ops_types.cu:20-49) -------------------- */

/* `path` = attr mul_map_file: raw little-endian uint16[65536], no header; NULL or "" gives
 * the exact product table.  `num_bits` = attr num_bits, must be 8.  Short or missing file:
 * AXC_INVALID_ARGUMENT ("ApproxTF: Couldn't read the lookup table!"). */
int axc_table_create_from_file(const char *path, int num_bits, axc_table **out);
int axc_table_create_from_memory(const uint16_t *lut65536, axc_table **out);
int axc_table_create_exact(axc_table **out);
void axc_table_destroy(axc_table *table);
/* Weight tuning of the first-generation op (attribute AxTune of AxConv2D, on by default there;
 * ApproximateSelector::init, tf1/axqconv/approximate_selector.h:46-78): out[i][w] = in[i][w2(w)], where w2(w) is
 * the weight column whose entries are closest to the exact products i*w in summed absolute error; among equally
 * good columns w itself wins, else the lowest index.  Host arithmetic on uint16[65536] arrays (index = a*256 + w);
 * `in` and `out` may be the same array.  Feed the result to axc_table_create_from_memory. */
int axc_table_tune_weights(const uint16_t *in65536, uint16_t *out65536);
/* Host copy of the 65536 entries (owned by the table). */
int axc_table_host_data(const axc_table *table, const uint16_t **out);
/* Uploads the 128 KiB replica for `device` if it is not there yet (blocking, once per
 * device) and, on the first use of a device by this library, runs a one-thread probe kernel that records where a
 * CTA's shared-memory window starts and ends there (the kernels place the table at fixed window addresses; a device
 * whose window does not fit makes every forward call return AXC_INTERNAL instead of launching).  axc_*_forward
 * does both lazily; call this first to keep them out of a timed or captured region. */
int axc_table_ensure_device(axc_table *table, int device);

/* ---- geometry: ComputeApproxConv2DDimensions (tf2/src/approx_nn_conv_ops.cpp:311-404) */
/* out4 = {n, out_h, out_w, out_c}; for the depthwise form out_c = c * cout. */
int axc_conv2d_output_dims(const axc_conv_desc *desc, int64_t out4[4]);
int axc_depthwise_conv2d_output_dims(const axc_conv_desc *desc, int64_t out4[4]);

/* Device scratch a forward call needs; stands in for the reference's allocate_temp buffers
 * (tf2/src/approx_nn_conv_ops.cpp:590-617).  The caller allocates it, 256-byte aligned.
 * For the dense op it holds the filter's lookup plan (quantised filter copy, table image, per-lane lookup
 * schedule, filter sums) and the fallback kernel's filter program.  The plan is rebuilt only when the buffer does not
 * already hold the plan of this very filter (values, ranges, table): keep one buffer per layer between
 * calls, leave it untouched, and the preparation is paid once; a fresh or recycled buffer is always safe
 * (its first 256 bytes decide), only slower.  One buffer serves one stream at a time. */
int axc_conv2d_workspace_bytes(const axc_conv_desc *desc, size_t *bytes);
int axc_depthwise_conv2d_workspace_bytes(const axc_conv_desc *desc, size_t *bytes);
/* Reads back {rebuilt in the last call, fallback kernel in use, kernel status (0 = fine), schedule steps per
 * ideal step in per-mille} of the plan in a dense workspace.  Blocks until `stream` is idle.  Diagnostics only;
 * no counterpart in the reference. */
int axc_conv2d_plan_info(const void *workspace, int32_t out4[4], int device, void *stream);

/* ---- forward: ApproxConv2DOp::Compute + LaunchApproxConv2DOp<GPUDevice>
 *      (tf2/src/approx_nn_conv_ops.cpp:420-460, 510-664) with the quantisation state of
 *      Update() (tf2/src/approx_ops_types.h:158-197) passed by value --------------------
 * in_min/in_max/f_min/f_max are the op's host-memory scalar inputs 2..5.
 * An output with zero elements returns AXC_OK without launching anything (:449-450).
 * Once the table replica is on the device (axc_table_ensure_device, or an earlier call) the workspace-taking forward
 * calls of this header (axc_conv2d_forward*, axc_depthwise_conv2d_forward, axc_depthwise_conv2d_forward_fused,
 * axc_qconv2d_forward) only enqueue kernels and memsets on `stream`: they may be captured into a CUDA graph and
 * replayed with the same buffers (tests/test_gpu_networks.py::test_forward_as_cuda_graph). */
int axc_conv2d_forward(axc_table *table, const axc_conv_desc *desc,
                       const float *input, const float *filter,
                       float in_min, float in_max, float f_min, float f_max,
                       float *output, void *workspace, size_t workspace_bytes,
                       const axc_debug_out *debug, int device, void *stream);

/* Steps of the op's callers that can ride along with the call: the bias and the activation of the reference's
 * Keras layer (tf2/python/keras/layers/fake_approx_convolutional.py:245-261), the shortcut of a residual block, and
 * the ReLU of the layer that PRODUCED this call's input.
 *   output side:  y = conv;  if (bias) y += bias[channel];  if (residual) y += residual[same index];
 *                 if (relu) y = max(y, 0)   - each a separately rounded fp32 operation, i.e. the bits of the same steps
 *                 done by separate kernels.  The dense op runs them as one extra pass over the output (inside the lookup
 *                 kernels even two instructions per output cost more than that pass); the depthwise kernels in place.
 *   input side:   input_relu != 0: every input element counts as max(x, 0) - applied by the kernels' loaders to the raw
 *                 value, before quantisation and patch sum, at no cost to the lookups.  A chain conv -> ReLU -> conv
 *                 can thus leave the ReLU to the second convolution and never write the activated tensor.
 * bias: [out channels] on the device or NULL; residual: a tensor of the output's shape on the device or NULL. */
typedef struct {
    const float *bias;
    const float *residual;
    int32_t relu;
    int32_t input_relu;
} axc_epilogue;
/* axc_conv2d_forward (ranges == NULL: the four host scalars count) or axc_conv2d_forward_device_ranges
 * (ranges != NULL) with a fused epilogue (NULL = none). */
int axc_conv2d_forward_fused(axc_table *table, const axc_conv_desc *desc, const float *input, const float *filter,
                             float in_min, float in_max, float f_min, float f_max, const float *ranges,
                             const axc_epilogue *epilogue, float *output, void *workspace, size_t workspace_bytes,
                             const axc_debug_out *debug, int device, void *stream);
int axc_depthwise_conv2d_forward_fused(axc_table *table, const axc_conv_desc *desc, const float *input,
                                       const float *filter, float in_min, float in_max, float f_min, float f_max,
                                       const axc_epilogue *epilogue, float *output, void *workspace,
                                       size_t workspace_bytes, const axc_debug_out *debug, int device, void *stream);

/* The shortcut step of a residual block on its own: out[i] = out[i] + residual[i], then max(., 0) if relu - one pass
 * over `count` floats (the pass axc_conv2d_forward_fused runs after the convolution, without a bias). */
int axc_add_residual(float *out, const float *residual, size_t count, int relu, int device, void *stream);

/* Max pooling of an NHWC fp32 tensor with a k x k window, stride `stride` and TensorFlow's SAME padding (taps outside
 * the image do not take part): out[n, oh, ow, c], oh = ceil(h / stride).  Not part of the op; the pooling step between
 * the stem and the first residual block of the ResNet workloads, kept in NHWC so that no layout copy is needed.
 * Max pooling commutes with ReLU, so a pending ReLU of the producing layer may be applied by the consumer as usual. */
int axc_max_pool_same(const float *input, float *output, int n, int h, int w, int c, int k, int stride, int device,
                      void *stream);

/* Same op with the four range scalars read from DEVICE memory: `ranges` = {input_min, input_max, filter_min,
 * filter_max}, four floats on `device`, typically written by the reductions that precede the op in the
 * reference's Keras wrapper (tf2/python/keras/layers/fake_approx_convolutional.py:233-242).  The quantisation
 * parameters are derived on the device with the host's arithmetic, so nothing waits for the host; the reference
 * pins these inputs to host memory (tf2/src/approx_nn_conv_ops.cpp:691-694), which costs a device-to-host
 * synchronisation per layer.  Results are bit-identical to axc_conv2d_forward with the same four values. */
int axc_conv2d_forward_device_ranges(axc_table *table, const axc_conv_desc *desc,
                                     const float *input, const float *filter, const float *ranges,
                                     float *output, void *workspace, size_t workspace_bytes,
                                     const axc_debug_out *debug, int device, void *stream);

/* ---- batch sharding over the GPUs of one box (no counterpart in the reference, which drives one GPU) ----------
 * Every output pixel depends on its own image only, so a batch is cut into contiguous NHWC slabs, one per shard; the
 * shards share nothing but the table handle (one 128 KiB replica per device) and the four range scalars, and no
 * collective sits on the compute path.  One shard = the tensors of one slab on one device with a stream and a
 * workspace of their own (axc_conv2d_workspace_bytes for a desc with n = the shard's images). */
typedef struct {
    int32_t device;
    int32_t n;                 /* images in this slab */
    const float *input;        /* [n,h,w,c] on `device` */
    const float *filter;       /* this device's copy of the filter */
    float *output;             /* [n,oh,ow,cout] on `device` */
    void *workspace;
    size_t workspace_bytes;
    void *stream;              /* cudaStream_t of `device` */
} axc_shard;
/* Enqueues axc_conv2d_forward for every shard (desc->n is ignored, the shard's n counts); the launches are
 * asynchronous, so one host thread keeps all GPUs busy.  Stops at the first shard that fails, stores its index in
 * *failed_shard (if not NULL; -1 when all were accepted) and returns that shard's status; shards before it are
 * already in flight and stay valid. */
int axc_conv2d_forward_sharded(axc_table *table, const axc_conv_desc *desc, const axc_shard *shards, int32_t nshards,
                               float in_min, float in_max, float f_min, float f_max, int32_t *failed_shard);
/* Optional gather of the shards' outputs into one contiguous [sum n, oh, ow, cout] tensor `dst` on `dst_device`:
 * one peer copy per shard, each enqueued on the shard's own stream (so it follows that shard's convolution), slab
 * order = shard order.  `image_bytes` = bytes of one image's output.  In a one-process-per-GPU deployment the same
 * step is an NCCL all-gather (the Python package's parallel.gather_outputs). */
int axc_gather_outputs(const axc_shard *shards, int32_t nshards, size_t image_bytes, void *dst, int32_t dst_device);

/* Depthwise variant (new: the reference rejects grouped shapes,
 * tf2/src/approx_nn_conv_ops.cpp:229-232).  filter [kh,kw,c,mult] in TensorFlow's
 * DepthwiseConv2dNative layout, output channel c*mult + m, same quantiser, table
 * indexing and dequantisation with K = kh*kw. */
int axc_depthwise_conv2d_forward(axc_table *table, const axc_conv_desc *desc,
                                 const float *input, const float *filter,
                                 float in_min, float in_max, float f_min, float f_max,
                                 float *output, void *workspace, size_t workspace_bytes,
                                 const axc_debug_out *debug, int device, void *stream);

/* Depthwise forward for callers that must not allocate device memory - an op kernel inside a framework
 * whose allocator has reserved the whole GPU up front (a plugin's own cudaMalloc then fails or steals from
 * the pool), or a serving loop that cannot afford cudaMalloc's implicit device-wide synchronisation.  It has
 * no counterpart in the reference.  Same arithmetic and results as axc_depthwise_conv2d_forward, but no
 * workspace argument: the scratch is a 1 MiB array that every GPU using this library carries until the
 * process exits.  Limits and rules:
 *   - the scratch a call needs - what axc_depthwise_conv2d_workspace_bytes() reports: about 6 bytes per filter
 *     element, 4 bytes per output channel and under 1 KiB of padding - must fit in 1 MiB (3x3 filters: up to
 *     about 17 000 channels), else AXC_INVALID_ARGUMENT; nothing is launched;
 *   - the table replica must already be on `device`: call axc_table_ensure_device() beforehand (that call
 *     allocates 128 KiB); otherwise AXC_INTERNAL;
 *   - the first call on a device looks up the array's device address; make that call before any stream
 *     capture starts; `device` must be below 64 (the addresses are remembered in a fixed table), else
 *     AXC_INVALID_ARGUMENT;
 *   - all calls on a device share the one array and each call overwrites what the previous one left, so
 *     two calls may not be in flight on the same GPU at the same time (different streams or threads): they
 *     would race on the scratch.  Nothing in it has to be cleared by the caller: every call rewrites the
 *     part it reads, including the status word, before using it.
 * No cudaMalloc/cudaFree or other allocating routine is called. */
int axc_depthwise_conv2d_forward_noalloc(axc_table *table, const axc_conv_desc *desc,
                                         const float *input, const float *filter,
                                         float in_min, float in_max, float f_min, float f_max,
                                         float *output, int device, void *stream);

/* ---- quantised operands in, int32 sums out: the contract of the reference's first-generation op AxConv2D
 *      (registration tf1/axqconv/axqconv.cc:66-94, arithmetic :197-263) ------------------------------------------
 * qinput [n,h,w,c] and qfilter [kh,kw,c,cout] are uint8 codes; every product of the integer convolution is
 * LUT[a][b], and the int32 result carries the reference's zero-point corrections
 *     output = sum_l ( LUT[a_l][b_l] - a_l*filter_offset - b_l*input_offset + input_offset*filter_offset ),
 * a tap outside the image counting as a_l = input_offset modulo 256 (the functor stores the offset into its uint8
 * operand type, :203-214; the zero-point terms use the offset as it is).  With both offsets 0 the output is the plain
 * table sum.  axc_quantized_zero_point gives the reference's offset for a float range; it lies outside 0..255 when
 * the range does not contain 0.  Offsets so large that K * max(|input_offset|, 255) * max(|filter_offset|, 255)
 * exceeds int32 return AXC_INVALID_ARGUMENT (the reference's int32 total would overflow).  As in the
 * reference op the strides must be equal and the dilation 1 (AXC_INVALID_ARGUMENT otherwise, :305-326); shapes on
 * which the reference functor would place the window differently from TensorFlow's padding rule (stride larger
 * than the window by two or more, :153-163) return AXC_UNIMPLEMENTED.  The table sums are computed by the kernels
 * of axc_conv2d_forward; the workspace additionally holds an fp32 image of both operands. */
int axc_qconv2d_workspace_bytes(const axc_conv_desc *desc, size_t *bytes);
int axc_qconv2d_forward(axc_table *table, const axc_conv_desc *desc, const uint8_t *qinput, const uint8_t *qfilter,
                        int32_t input_offset, int32_t filter_offset, int32_t *output, void *workspace,
                        size_t workspace_bytes, int device, void *stream);
/* The uint8 code of the real value 0 in [range_min, range_max]: FloatToQuantizedUnclamped<quint8>(0.0f, ...)
 * (tf1/axqconv/quantization_utils.h:49-64; the op's offsets, tf1/axqconv/axqconv.cc:365-368). */
int axc_quantized_zero_point(float range_min, float range_max, int32_t *offset);
/* out2 = {min_output, max_output} of the op: QuantizationRangeForMultiplication<quint8, quint8, qint32>
 * (tf1/axqconv/quantization_utils.h:116-140, tf1/axqconv/axqconv.cc:429-441). */
int axc_quantized_output_range(float min_a, float max_a, float min_b, float max_b, float out2[2]);

/* Status word the depthwise kernels leave in their scratch: 0 = fine, 1 = a kernel found its shared-memory layout
 * broken and returned without writing the output, 3 = a bulk copy into shared memory did not arrive within its
 * time limit.  `workspace` = the buffer of the forward call, or NULL for the built-in scratch of
 * axc_depthwise_conv2d_forward_noalloc.  Blocks until `stream` is idle.  The forward calls themselves are
 * asynchronous: AXC_OK from them means that the launches were accepted; what the kernels found is read here and, for
 * the dense op, with axc_conv2d_plan_info.  No counterpart in the reference, which never checks a CUDA result. */
int axc_depthwise_conv2d_status(const axc_conv_desc *desc, const void *workspace, int32_t *status, int device, void *stream);

/* ---- the steps that precede the op in the reference's Keras wrapper, on the device
 *      (tf2/python/keras/layers/fake_approx_convolutional.py:233-242: reduce_min / reduce_max of the tensor, then
 *      FakeQuantWithMinMaxVars) --------------------------------------------------------------------------------- */
/* range2 (device, two floats) = {min, max} over the `count` floats at x: one reduction kernel (plus a two-thread
 * kernel that resets range2).  NaNs are skipped.  count == 0 leaves {+inf, -inf}.  Write input and filter ranges
 * into the two halves of one four-float buffer and hand it to axc_conv2d_forward_device_ranges. */
int axc_tensor_range(const float *x, size_t count, float *range2, int device, void *stream);
/* out[i] = x[i] clamped to the nudged range and snapped to its 256-level grid: the forward of TensorFlow's
 * FakeQuantWithMinMaxVars with num_bits = 8, with the range read from device memory (range2 = {min, max}); the
 * nudging is the op's own (tf2/src/approx_ops_types.h:29-49), operation by operation.  out may equal x. */
int axc_fake_quant(const float *x, size_t count, const float *range2, float *out, int device, void *stream);

/* ---- quantisation parameters: Nudge + UpdateVarQuantProps
 *      (tf2/src/approx_ops_types.h:29-49, 135-152).  out3 = {scale, 1/scale, nudged_min}. */
int axc_quant_props(float min_value, float max_value, float out3[3]);

/* ---- diagnostics ------------------------------------------------------------------- */
const char *axc_status_string(int status);
/* cudaError_t of the most recent AXC_CUDA_ERROR on the calling thread (0 if none). */
int axc_last_cuda_error(void);
/* Number of kernels this library has launched in the calling process (monotonic). */
uint64_t axc_launch_count(void);
/* Debug flavour only (libaxconv_check.so, built with -DAXC_BOUNDS_CHECK): every shared-memory address the kernels
 * compute and every global index they form is checked before use; a violation is counted and skipped, never a trap.
 * out4 = {violations since the last call, site number of the first, its offending value: low word, high word};
 * reading clears the record.  Blocks until the device is idle.  In the normal build: AXC_UNIMPLEMENTED.  No
 * counterpart in the reference. */
int axc_debug_bounds_record(int device, uint32_t out4[4]);

/* Measures what one SM sustains in conflict-free 16-bit shared-memory loads - the operation a table MAC of the
 * dense kernels costs (the reference does the same lookup through a texture fetch,
 * tf2/src/cuda/approx_nn_conv_kernels.cu:471-472) - in lookups per clock and SM; 32 by the construction of the
 * hardware.  One short kernel on every SM, then a blocking read-back.  `scratch`: device memory, 256-byte aligned,
 * at least 256 + 8 * (number of SMs) bytes.  Diagnostics for roofline reports; no counterpart in the reference. */
int axc_measure_lookup_peak(int device, void *scratch, size_t scratch_bytes, void *stream,
                            double *lookups_per_clk_per_sm);

#ifdef __cplusplus
}
#endif
#endif /* AXCONV_H */
