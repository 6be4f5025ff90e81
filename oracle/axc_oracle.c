/*
 * TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 *
 * CPU restatement of the table-driven convolution of ehw-fit/tf-approximate
 * (tf2 generation).  It exists only as the checker for the CUDA path and as
 * the timed CPU baseline; the shipped library never links or calls it.
 *
 * Parity status: the arithmetic of this file is pinned twice,
 *   - against the reference's own kernel translation unit compiled from where
 *     it lies (oracle/Makefile -> oracle/_ref/libaxc_ref.so), on seeded
 *     inputs, bit for bit (tests/test_oracle_vs_ref.py);
 *   - against the reference's golden material: the exact-product table file
 *     of its op test and its 36 multiplier tables (tests/golden/).
 * The depthwise variant has no counterpart in the reference ("parity
 * unpinned"): it applies the same per-MAC rule to a grouped shape the
 * reference rejects (tf2/src/approx_nn_conv_ops.cpp:229-232).
 *
 * Every float operation is a separately rounded binary32 operation
 * (build with -O2 -ffp-contract=off, no -ffast-math).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define AXO_OK 0
#define AXO_INVALID_ARGUMENT 3
#define AXO_UNIMPLEMENTED 12

#define AXO_PAD_SAME 0
#define AXO_PAD_VALID 1

typedef struct {
    int n, h, w, c;          /* input, NHWC                                  */
    int kh, kw, cout;        /* filter [kh,kw,c,cout]; depthwise: cout=mult  */
    int stride_h, stride_w;
    int dil_h, dil_w;
    int padding;             /* AXO_PAD_SAME / AXO_PAD_VALID                 */
} axo_conv_desc;

typedef struct {
    float scale, inv_scale, offset;
} axo_var_quant;

typedef struct {
    axo_var_quant input, filter;
    float s1s2, m1, m2, m1m2;
} axo_quant;

/* tf2/src/approx_ops_types.h:29-49 (Nudge) and :135-152 (UpdateVarQuantProps):
 * scale=(max-min)/255, zero point clamped/rounded half away from zero, stored
 * as uint16, nudged_min=(0-zp)*scale; an all-zero range gives all-zero props. */
void axo_var_quant_props(float min_v, float max_v, axo_var_quant *q)
{
    float scale = 0.0f, inv = 0.0f, nudged_min = 0.0f;
    if (min_v != 0.0f || max_v != 0.0f) {
        const float qmin = 0.0f, qmax = 255.0f;
        scale = (max_v - min_v) / (qmax - qmin);
        const float zp_from_min = qmin - min_v / scale;
        uint16_t zp;
        if (zp_from_min < qmin)
            zp = 0;
        else if (zp_from_min > qmax)
            zp = 255;
        else
            zp = (uint16_t)roundf(zp_from_min);
        /* (0 - zp) first, then the product: kept apart so that a zero zero-point gives +0.0 as in the
         * reference (an optimiser folding the subtraction into the product would give -0.0) */
        volatile float zp_f = (float)zp, zero = qmin;
        volatile float neg_zp = zero - zp_f;
        nudged_min = neg_zp * scale;
        inv = 1.0f / scale;
    }
    q->scale = scale;
    q->inv_scale = inv;
    q->offset = nudged_min;
}

/* tf2/src/approx_ops_types.h:158-197 (Update). */
void axo_quant_props(float in_min, float in_max, float f_min, float f_max, axo_quant *q)
{
    axo_var_quant_props(in_min, in_max, &q->input);
    axo_var_quant_props(f_min, f_max, &q->filter);
    q->s1s2 = q->input.scale * q->filter.scale;
    q->m1 = q->input.offset;
    q->m2 = q->filter.offset;
    q->m1m2 = q->m1 * q->m2;
}

/* Element quantiser, tf2/src/approx_nn_conv_kernels.cpp:293 and :243:
 * uint8(((x - offset) * inv) + 0.5f), truncating cast.  The reference cast is
 * undefined outside [0,256); this restatement and the CUDA op saturate there
 * (in-range inputs - the op's contract - are unaffected). */
static inline uint8_t axo_q(float x, float offset, float inv)
{
    const float d = x - offset;
    const float s = d * inv;
    const float v = s + 0.5f;
    if (!(v > 0.0f))
        return 0;
    if (v >= 255.0f)
        return 255;
    return (uint8_t)v;
}

uint8_t axo_quantize(float x, float offset, float inv) { return axo_q(x, offset, inv); }

/* tf2/src/approx_ops_types.h:112-117: empty file name -> exact product table,
 * index = (a << 8) | b. */
void axo_exact_table(uint16_t *lut)
{
    for (uint32_t i = 0; i < 65536u; ++i)
        lut[i] = (uint16_t)((i >> 8) * (i & 0xFFu));
}

/* tf2/src/approx_ops_types.h:205-216: raw little-endian uint16[65536], no
 * header; a short or missing file is InvalidArgument. */
int axo_load_table(const char *path, uint16_t *lut)
{
    memset(lut, 0, 65536u * sizeof(uint16_t));
    FILE *f = fopen(path, "rb");
    if (!f)
        return AXO_INVALID_ARGUMENT;
    size_t got = fread(lut, sizeof(uint16_t), 65536u, f);
    fclose(f);
    return got == 65536u ? AXO_OK : AXO_INVALID_ARGUMENT;
}

/* TF window arithmetic used by tf2/src/approx_nn_conv_ops.cpp:376-382
 * (GetWindowedOutputSizeVerboseV2): SAME -> ceil(in/stride) and
 * pad_before = max((out-1)*stride + (k-1)*dil + 1 - in, 0) / 2;
 * VALID -> ceil((in - (k-1)*dil) / stride), no padding. */
static int axo_window(int in, int k, int dil, int stride, int padding, int *out, int *pad_before)
{
    const int eff = (k - 1) * dil + 1;
    if (padding == AXO_PAD_VALID) {
        *out = (in - eff + stride) / stride;
        *pad_before = 0;
    } else if (padding == AXO_PAD_SAME) {
        *out = (in + stride - 1) / stride;
        int need = (*out - 1) * stride + eff - in;
        if (need < 0)
            need = 0;
        *pad_before = need / 2;
    } else {
        return AXO_UNIMPLEMENTED;
    }
    if (*out < 0)
        return AXO_INVALID_ARGUMENT;
    return AXO_OK;
}

int axo_out_dims(const axo_conv_desc *d, int *oh, int *ow, int *ph, int *pw)
{
    if (d->n < 0 || d->h < 0 || d->w < 0 || d->c < 0 || d->kh <= 0 || d->kw <= 0 || d->cout < 0 ||
        d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 || d->dil_w <= 0)
        return AXO_INVALID_ARGUMENT;
    int rc = axo_window(d->h, d->kh, d->dil_h, d->stride_h, d->padding, oh, ph);
    if (rc)
        return rc;
    return axo_window(d->w, d->kw, d->dil_w, d->stride_w, d->padding, ow, pw);
}

/* Patch builder, tf2/src/approx_nn_conv_kernels.cpp:260-296: element order
 * (kh, kw, c) with c fastest, zero outside the image, quantised bytes into
 * `a`, fp32 sum of the raw values (zeros included) in element order. */
static void axo_im2col(const axo_quant *q, const float *in, int c, int w, int h, int ow, int oh,
                       int kw, int kh, int pw, int ph, int sw, int sh, int dw, int dh,
                       int64_t po, int pc, uint8_t *a, float *a_sum)
{
    const int pl = c * kw * kh;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < pc; ++i) {
        const int64_t patch = po + i;
        const int out_b = (int)((patch / ow) / oh);
        const int out_h = (int)((patch / ow) % oh);
        const int out_w = (int)(patch % ow);
        float sum = 0.0f;
        uint8_t *row = a + (size_t)i * pl;
        for (int v = 0; v < pl; ++v) {
            const int off_h = v / (kw * c);
            const int off_w = (v / c) % kw;
            const int off_c = v % c;
            const int in_h = out_h * sh - ph + off_h * dh;
            const int in_w = out_w * sw - pw + off_w * dw;
            float value = 0.0f;
            if (in_h >= 0 && in_w >= 0 && in_h < h && in_w < w)
                value = in[(((size_t)out_b * h + in_h) * w + in_w) * c + off_c];
            row[v] = axo_q(value, q->input.offset, q->input.inv_scale);
            sum += value;
        }
        a_sum[i] = sum;
    }
}

/* Table GEMM + dequantisation, tf2/src/approx_nn_conv_kernels.cpp:215-256:
 * weight re-quantised for every MAC, fp32 running total in l order,
 * out = total*s1s2 + m2*aSum + m1*bSum - float(k)*m1m2 (left to right).
 * acc (exact integer sum) and out_exact (same epilogue on float(acc)) are
 * additions for the parity tests. */
static void axo_gemm(const axo_quant *q, const uint16_t *lut, int m, int n, int k,
                     const uint8_t *a, const float *b, const float *a_sum, const float *b_sum,
                     float *out_ref, float *out_exact, int32_t *acc)
{
#pragma omp parallel for schedule(static)
    for (int j = 0; j < n; ++j) {
        for (int i = 0; i < m; ++i) {
            float total = 0.0f;
            int64_t exact = 0;
            const uint8_t *arow = a + (size_t)i * k;
            for (int l = 0; l < k; ++l) {
                const uint32_t av = arow[l];
                const uint32_t bv = axo_q(b[(size_t)l * n + j], q->filter.offset, q->filter.inv_scale);
                const uint32_t cv = lut[(av << 8) | bv];
                total += (float)cv;
                exact += cv;
            }
            const size_t ci = (size_t)i * n + j;
            const float kf = (float)k;
            if (out_ref) {
                const float t0 = total * q->s1s2;
                const float t1 = q->m2 * a_sum[i];
                const float t2 = q->m1 * b_sum[j];
                const float t3 = kf * q->m1m2;
                out_ref[ci] = ((t0 + t1) + t2) - t3;
            }
            if (out_exact) {
                const float t0 = (float)exact * q->s1s2;
                const float t1 = q->m2 * a_sum[i];
                const float t2 = q->m1 * b_sum[j];
                const float t3 = kf * q->m1m2;
                out_exact[ci] = ((t0 + t1) + t2) - t3;
            }
            if (acc)
                acc[ci] = (int32_t)exact;
        }
    }
}

/* Fused form for 1x1 stride-1 and filter==image VALID shapes,
 * tf2/src/approx_nn_conv_kernels.cpp:167-211: both operands quantised in the
 * l loop, aSum and bSum accumulated sequentially in that loop. */
static void axo_gemm_combined(const axo_quant *q, const uint16_t *lut, int m, int n, int k,
                              const float *a, const float *b,
                              float *out_ref, float *out_exact, int32_t *acc)
{
#pragma omp parallel for schedule(static)
    for (int j = 0; j < n; ++j) {
        for (int i = 0; i < m; ++i) {
            float total = 0.0f, a_sum = 0.0f, b_sum = 0.0f;
            int64_t exact = 0;
            for (int l = 0; l < k; ++l) {
                const float av_f = a[(size_t)i * k + l];
                const uint32_t av = axo_q(av_f, q->input.offset, q->input.inv_scale);
                a_sum += av_f;
                const float bv_f = b[(size_t)l * n + j];
                const uint32_t bv = axo_q(bv_f, q->filter.offset, q->filter.inv_scale);
                b_sum += bv_f;
                const uint32_t cv = lut[(av << 8) | bv];
                total += (float)cv;
                exact += cv;
            }
            const size_t ci = (size_t)i * n + j;
            const float kf = (float)k;
            if (out_ref) {
                const float t0 = total * q->s1s2;
                const float t1 = q->m2 * a_sum;
                const float t2 = q->m1 * b_sum;
                const float t3 = kf * q->m1m2;
                out_ref[ci] = ((t0 + t1) + t2) - t3;
            }
            if (out_exact) {
                const float t0 = (float)exact * q->s1s2;
                const float t1 = q->m2 * a_sum;
                const float t2 = q->m1 * b_sum;
                const float t3 = kf * q->m1m2;
                out_exact[ci] = ((t0 + t1) + t2) - t3;
            }
            if (acc)
                acc[ci] = (int32_t)exact;
        }
    }
}

/* tf2/src/approx_nn_conv_kernels.cpp:300-306: per output channel sum of the
 * fp32 filter over (kh, kw, c).  Eigen leaves the order open; this restatement
 * sums in l order. */
static void axo_filter_sums(const float *filter, int k, int n, float *b_sum)
{
    for (int j = 0; j < n; ++j) {
        float s = 0.0f;
        for (int l = 0; l < k; ++l)
            s += filter[(size_t)l * n + j];
        b_sum[j] = s;
    }
}

/*
 * Forward pass with the reference's CPU dispatch
 * (tf2/src/approx_nn_conv_ops.cpp:70-206): 1x1 stride 1 -> fused form;
 * filter == image, dilation 1, VALID -> fused form; everything else im2col +
 * GEMM in chunks of 16 MiB / sizeof(float) patch elements (:118-124, :168-202).
 *
 * Optional outputs (NULL to skip):
 *   out_ref   fp32 [N,OH,OW,Cout]  reference arithmetic (fp32 running total)
 *   out_exact fp32 [N,OH,OW,Cout]  same epilogue on the exact integer sum
 *   acc       i32  [N,OH,OW,Cout]  exact integer sum of table entries
 *   qinput    u8   [N,H,W,C]       element-wise quantised input
 *   qfilter   u8   [KH*KW*C,Cout]  element-wise quantised filter
 *   pad_q     u8   [1]             quantised value of an out-of-image tap
 */
int axo_conv2d(const axo_conv_desc *d, const uint16_t *lut, const float *input, const float *filter,
               float in_min, float in_max, float f_min, float f_max,
               float *out_ref, float *out_exact, int32_t *acc,
               uint8_t *qinput, uint8_t *qfilter, uint8_t *pad_q, int nthreads)
{
    int oh, ow, ph, pw;
    int rc = axo_out_dims(d, &oh, &ow, &ph, &pw);
    if (rc)
        return rc;
#ifdef _OPENMP
    if (nthreads > 0)
        omp_set_num_threads(nthreads);
#else
    (void)nthreads;
#endif
    axo_quant q;
    axo_quant_props(in_min, in_max, f_min, f_max, &q);

    const int64_t k64 = (int64_t)d->kh * d->kw * d->c;
    const int n = d->cout;
    if (qinput) {
        const size_t cnt = (size_t)d->n * d->h * d->w * d->c;
        for (size_t i = 0; i < cnt; ++i)
            qinput[i] = axo_q(input[i], q.input.offset, q.input.inv_scale);
    }
    if (qfilter) {
        const size_t cnt = (size_t)k64 * n;
        for (size_t i = 0; i < cnt; ++i)
            qfilter[i] = axo_q(filter[i], q.filter.offset, q.filter.inv_scale);
    }
    if (pad_q)
        *pad_q = axo_q(0.0f, q.input.offset, q.input.inv_scale);

    const int64_t total_patches = (int64_t)d->n * oh * ow;
    if (total_patches == 0 || n == 0)
        return AXO_OK;

    if (d->kh == 1 && d->kw == 1 && d->stride_h == 1 && d->stride_w == 1) {
        axo_gemm_combined(&q, lut, (int)((int64_t)d->n * d->h * d->w), n, d->c,
                          input, filter, out_ref, out_exact, acc);
        return AXO_OK;
    }
    if (d->kh == d->h && d->kw == d->w && d->dil_h == 1 && d->dil_w == 1 && d->padding == AXO_PAD_VALID) {
        axo_gemm_combined(&q, lut, d->n, n, (int)((int64_t)d->h * d->w * d->c),
                          input, filter, out_ref, out_exact, acc);
        return AXO_OK;
    }

    const int64_t max_chunk = (16 * 1024 * 1024) / (int64_t)sizeof(float);
    if (k64 > max_chunk)
        return AXO_INVALID_ARGUMENT; /* "Patch too large for buffer" */
    const int k = (int)k64;
    const int64_t per_chunk = max_chunk / k;

    uint8_t *a = (uint8_t *)malloc((size_t)max_chunk);
    float *a_sum = (float *)malloc(sizeof(float) * (size_t)per_chunk);
    float *b_sum = (float *)malloc(sizeof(float) * (size_t)n);
    if (!a || !a_sum || !b_sum) {
        free(a); free(a_sum); free(b_sum);
        return AXO_INVALID_ARGUMENT;
    }
    axo_filter_sums(filter, k, n, b_sum);

    const int64_t per_image = (int64_t)oh * ow;
    for (int64_t i = 0; i < total_patches; i += per_chunk) {
        const int64_t batch = i / per_image;
        const int64_t patch_off = i % per_image;
        const int pc = (int)((per_chunk < total_patches - i) ? per_chunk : (total_patches - i));
        const float *in_b = input + (size_t)batch * d->h * d->w * d->c;
        axo_im2col(&q, in_b, d->c, d->w, d->h, ow, oh, d->kw, d->kh, pw, ph,
                   d->stride_w, d->stride_h, d->dil_w, d->dil_h, patch_off, pc, a, a_sum);
        const size_t o = (size_t)i * n;
        axo_gemm(&q, lut, pc, n, k, a, filter, a_sum, b_sum,
                 out_ref ? out_ref + o : NULL, out_exact ? out_exact + o : NULL, acc ? acc + o : NULL);
    }
    free(a); free(a_sum); free(b_sum);
    return AXO_OK;
}

/*
 * Independent cross-check: the direct seven-deep loop of
 * tf2/src/approx_nn_conv_ops_ref.cpp:231-317 (no dilation; centre-based
 * padding offsets :242-251; both operands quantised per MAC; patch sums
 * accumulated inside the loop, so bSum is sequential here).
 */
int axo_conv2d_direct(const axo_conv_desc *d, const uint16_t *lut, const float *input, const float *filter,
                      float in_min, float in_max, float f_min, float f_max, float *out)
{
    int oh, ow, ph, pw;
    int rc = axo_out_dims(d, &oh, &ow, &ph, &pw);
    if (rc)
        return rc;
    if (d->dil_h != 1 || d->dil_w != 1)
        return AXO_UNIMPLEMENTED;
    axo_quant q;
    axo_quant_props(in_min, in_max, f_min, f_max, &q);
    int left, top;
    if (d->padding == AXO_PAD_VALID) {
        left = ((ow - 1) * d->stride_w + d->kw - d->w + 1) / 2;
        top = ((oh - 1) * d->stride_h + d->kh - d->h + 1) / 2;
    } else {
        left = ((ow - 1) * d->stride_w + d->kw - d->w) / 2;
        top = ((oh - 1) * d->stride_h + d->kh - d->h) / 2;
    }
    const int C = d->c, F = d->cout;
    for (int b = 0; b < d->n; ++b)
        for (int oy = 0; oy < oh; ++oy)
            for (int ox = 0; ox < ow; ++ox)
                for (int oc = 0; oc < F; ++oc) {
                    const int x0 = ox * d->stride_w - left;
                    const int y0 = oy * d->stride_h - top;
                    float total = 0.0f, in_tot = 0.0f, f_tot = 0.0f;
                    for (int fy = 0; fy < d->kh; ++fy)
                        for (int fx = 0; fx < d->kw; ++fx)
                            for (int ic = 0; ic < C; ++ic) {
                                const int ix = x0 + fx, iy = y0 + fy;
                                float iv = 0.0f;
                                if (ix >= 0 && ix < d->w && iy >= 0 && iy < d->h)
                                    iv = input[(((size_t)b * d->h + iy) * d->w + ix) * C + ic];
                                const float fv = filter[(((size_t)fy * d->kw + fx) * C + ic) * F + oc];
                                in_tot += iv;
                                f_tot += fv;
                                const uint32_t qa = axo_q(iv, q.input.offset, q.input.inv_scale);
                                const uint32_t qb = axo_q(fv, q.filter.offset, q.filter.inv_scale);
                                total += (float)lut[(qa << 8) | qb];
                            }
                    const float kf = (float)(d->kh * d->kw * C);
                    const float t0 = total * q.s1s2;
                    const float t1 = q.m2 * in_tot;
                    const float t2 = q.m1 * f_tot;
                    const float t3 = kf * q.m1m2;
                    out[(((size_t)b * oh + oy) * ow + ox) * F + oc] = ((t0 + t1) + t2) - t3;
                }
    return AXO_OK;
}

/*
 * First-generation op AxConv2D: quantised uint8 operands in, int32 sums out.
 * Restates ReferenceConvFunctor::operator() of tf1/axqconv/axqconv.cc:132-263
 * loop for loop: window origin from the functor's own offsets (:153-163), a tap
 * outside the image counts as input_offset stored into the uint8 operand type,
 * i.e. modulo 256 (:203-214), every product is a table entry (:232) and carries
 * the zero-point terms with the unwrapped offsets (:241-246); offset_output = 0,
 * mult_output = 1, shift_output = 0 (:369-371) leave the total as the output.
 * Pin: the op's own Compute(), compiled from the reference checkout against
 * stand-in headers (ref_axq_driver.cpp, _ref/libaxq_ref.so), on random shapes,
 * ranges and multipliers, bit for bit (tests/test_oracle_vs_ref.py).
 */
int axo_qconv2d(const axo_conv_desc *d, const uint16_t *lut, const uint8_t *qin, const uint8_t *qf, int input_offset,
                int filter_offset, int32_t *out)
{
    int oh, ow, ph, pw;
    int rc = axo_out_dims(d, &oh, &ow, &ph, &pw);
    if (rc)
        return rc;
    if (d->dil_h != 1 || d->dil_w != 1 || d->stride_h != d->stride_w)
        return AXO_INVALID_ARGUMENT;
    const int stride = d->stride_h;
    int left, top;
    if (d->padding == AXO_PAD_VALID) {
        left = ((ow - 1) * stride + d->kw - d->w + 1) / 2;
        top = ((oh - 1) * stride + d->kh - d->h + 1) / 2;
    } else {
        left = ((ow - 1) * stride + d->kw - d->w) / 2;
        top = ((oh - 1) * stride + d->kh - d->h) / 2;
    }
    const int C = d->c, F = d->cout;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < d->n; ++b)
        for (int oy = 0; oy < oh; ++oy)
            for (int ox = 0; ox < ow; ++ox)
                for (int oc = 0; oc < F; ++oc) {
                    const int x0 = ox * stride - left;
                    const int y0 = oy * stride - top;
                    int32_t total = 0;
                    for (int fy = 0; fy < d->kh; ++fy)
                        for (int fx = 0; fx < d->kw; ++fx)
                            for (int ic = 0; ic < C; ++ic) {
                                const int ix = x0 + fx, iy = y0 + fy;
                                int32_t a = (uint8_t)input_offset;
                                if (ix >= 0 && ix < d->w && iy >= 0 && iy < d->h)
                                    a = qin[(((size_t)b * d->h + iy) * d->w + ix) * C + ic];
                                const int32_t w = qf[(((size_t)fy * d->kw + fx) * C + ic) * F + oc];
                                const int32_t axm = lut[(a << 8) | w];
                                total += axm - a * filter_offset - w * input_offset + input_offset * filter_offset;
                            }
                    out[(((size_t)b * oh + oy) * ow + ox) * F + oc] = total;
                }
    return AXO_OK;
}

/*
 * Weight tuning of the first-generation op (attribute AxTune, on by default):
 * ApproximateSelector::init, tf1/axqconv/approximate_selector.h:46-78.  Column w
 * of the table is replaced by the column w2 whose entries are closest to the exact
 * products i * w in summed absolute error; among equally good columns w itself
 * wins, else the lowest index.  in/out: uint16[65536], index = data * 256 + weight.
 */
void axo_tune_table(const uint16_t *in, uint16_t *out)
{
    for (int w = 0; w < 256; ++w) {
        int wpos = -1;
        int werr = 0;
        for (int w2 = 0; w2 < 256; ++w2) {
            int sumerr = 0;
            for (int i = 0; i < 256; ++i)
                sumerr += abs(i * w - (int)in[i * 256 + w2]);
            if (sumerr < werr || (werr == sumerr && w2 == w) || wpos < 0) {
                werr = sumerr;
                wpos = w2;
            }
        }
        for (int i = 0; i < 256; ++i)
            out[i * 256 + w] = in[i * 256 + wpos];
    }
}

/* FloatToQuantizedUnclamped<quint8>(0.0f, min, max), tf1/axqconv/quantization_utils.h:49-64. */
int32_t axo_quantized_zero_point(float range_min, float range_max)
{
    if (range_min == range_max)
        return 0;
    const int64_t number_of_steps = (int64_t)1 << 8;
    const double range_adjust = (number_of_steps / (number_of_steps - 1.0));
    const double range = ((range_max - range_min) * range_adjust);
    const double range_scale = (number_of_steps / range);
    int64_t quantized = (int64_t)(round(0.0f * range_scale) - round(range_min * range_scale));
    return (int32_t)quantized;
}

/* QuantizationRangeForMultiplication<quint8, quint8, qint32>, tf1/axqconv/quantization_utils.h:116-140. */
void axo_quantized_output_range(float min_a, float max_a, float min_b, float max_b, float *min_c, float *max_c)
{
    const float a_level = (max_a - min_a) / (int64_t)(255 - 0);
    const float b_level = (max_b - min_b) / (int64_t)(255 - 0);
    const int64_t c_highest = 2147483647ll, c_lowest = -2147483647ll - 1;
    const float c_level = a_level * b_level;
    *min_c = c_level * c_lowest;
    *max_c = c_level * c_highest;
}

/*
 * Depthwise variant (no reference counterpart; the reference rejects grouped
 * shapes, tf2/src/approx_nn_conv_ops.cpp:229-232).  Filter [KH,KW,C,mult]
 * (TensorFlow DepthwiseConv2dNative layout), output channel c*mult+m.
 * Same quantiser, table index (qa<<8)|qb, tap order (kh,kw), same epilogue
 * with K = KH*KW; aSum and bSum are sequential fp32 sums in tap order.
 */
int axo_depthwise_conv2d(const axo_conv_desc *d, const uint16_t *lut, const float *input, const float *filter,
                         float in_min, float in_max, float f_min, float f_max,
                         float *out_ref, float *out_exact, int32_t *acc, int nthreads)
{
    int oh, ow, ph, pw;
    int rc = axo_out_dims(d, &oh, &ow, &ph, &pw);
    if (rc)
        return rc;
#ifdef _OPENMP
    if (nthreads > 0)
        omp_set_num_threads(nthreads);
#else
    (void)nthreads;
#endif
    axo_quant q;
    axo_quant_props(in_min, in_max, f_min, f_max, &q);
    const int C = d->c, MUL = d->cout;
    const int k = d->kh * d->kw;
    const float kf = (float)k;
    const int64_t rows = (int64_t)d->n * oh;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const int b = (int)(r / oh), oy = (int)(r % oh);
        for (int ox = 0; ox < ow; ++ox)
            for (int c = 0; c < C; ++c)
                for (int m = 0; m < MUL; ++m) {
                    float total = 0.0f, a_sum = 0.0f, b_sum = 0.0f;
                    int64_t exact = 0;
                    for (int fy = 0; fy < d->kh; ++fy)
                        for (int fx = 0; fx < d->kw; ++fx) {
                            const int iy = oy * d->stride_h - ph + fy * d->dil_h;
                            const int ix = ox * d->stride_w - pw + fx * d->dil_w;
                            float iv = 0.0f;
                            if (ix >= 0 && ix < d->w && iy >= 0 && iy < d->h)
                                iv = input[(((size_t)b * d->h + iy) * d->w + ix) * C + c];
                            const float fv = filter[(((size_t)fy * d->kw + fx) * C + c) * MUL + m];
                            a_sum += iv;
                            b_sum += fv;
                            const uint32_t qa = axo_q(iv, q.input.offset, q.input.inv_scale);
                            const uint32_t qb = axo_q(fv, q.filter.offset, q.filter.inv_scale);
                            const uint32_t cv = lut[(qa << 8) | qb];
                            total += (float)cv;
                            exact += cv;
                        }
                    const size_t oi = (((size_t)b * oh + oy) * ow + ox) * ((size_t)C * MUL) + (size_t)c * MUL + m;
                    if (out_ref) {
                        const float t0 = total * q.s1s2, t1 = q.m2 * a_sum, t2 = q.m1 * b_sum, t3 = kf * q.m1m2;
                        out_ref[oi] = ((t0 + t1) + t2) - t3;
                    }
                    if (out_exact) {
                        const float t0 = (float)exact * q.s1s2, t1 = q.m2 * a_sum, t2 = q.m1 * b_sum, t3 = kf * q.m1m2;
                        out_exact[oi] = ((t0 + t1) + t2) - t3;
                    }
                    if (acc)
                        acc[oi] = (int32_t)exact;
                }
    }
    return AXO_OK;
}

int axo_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
