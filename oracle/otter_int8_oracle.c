/* CPU restatement of the reference's int8 convolution path — TEST INFRASTRUCTURE ONLY.
 * See otter_int8_oracle.h for what each function follows in the reference and for the parity status
 * (pinned against the compiled reference; the reference itself has no golden vectors for this path).
 *
 * Compile with -ffp-contract=off: every fused multiply-add below is written as fmaf() on purpose,
 * and every separate multiply / add must stay separate.
 */
#include "otter_int8_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Tensor/VecIntrinsic.hpp:71-95 (add ±0.5, cvttps, packs to s16, min 127 / max -127)
 * Tensor/QuantizeX86.cpp:18-23 (round(), clamp). */
int8_t orc_float2int8(float v, int rounding) {
    int32_t i;
    if (rounding == ORC_ROUND_HALF_AWAY) {
        float r = roundf(v);
        if (!(r > -2147483648.0f && r < 2147483648.0f)) return r > 0 ? 127 : -127;
        i = (int32_t)r;
    } else {
        float adj = v + copysignf(0.5f, v);
        /* cvttps yields INT_MIN when out of range; packs_epi32 then saturates to -32768 -> -127 */
        if (!(adj > -2147483648.0f && adj < 2147483648.0f)) return -127;
        i = (int32_t)adj; /* truncation */
    }
    if (i > 127) return 127;
    if (i < -127) return -127;
    return (int8_t)i;
}

void orc_scale_in(const float* w_scales, int cout, float in_scale0, float* scale_in) {
    for (int p = 0; p < cout; ++p)
        scale_in[p] = w_scales[p] == 0.f ? 0.f : 1.f / (in_scale0 * w_scales[p]);
}

void orc_quantize(const float* x, int n, int c, int h, int w, const float* scales, int n_scales,
                  int rounding, int8_t* out) {
    const long hw = (long)h * w;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b)
        for (int q = 0; q < c; ++q) {
            const float s = n_scales == 1 ? scales[0] : scales[q];
            const float* src = x + ((long)b * c + q) * hw;
            int8_t* dst = out + ((long)b * c + q) * hw;
            for (long i = 0; i < hw; ++i) dst[i] = orc_float2int8(src[i] * s, rounding);
        }
}

void orc_conv_s32(const int8_t* x, int n, int cin, int h, int w, const int8_t* wt, int cout,
                  int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups, int32_t* acc) {
    const int oh = (h + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    const int ow = (w + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    const int cin_g = cin / groups, cout_g = cout / groups;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b)
        for (int o = 0; o < cout; ++o) {
            const int g = o / cout_g;
            const int8_t* wo = wt + (long)o * cin_g * kh * kw;
            int32_t* dst = acc + ((long)b * cout + o) * oh * ow;
            for (int oy = 0; oy < oh; ++oy)
                for (int ox = 0; ox < ow; ++ox) {
                    int32_t sum = 0;
                    for (int ci = 0; ci < cin_g; ++ci) {
                        const int8_t* xc = x + ((long)b * cin + g * cin_g + ci) * h * w;
                        const int8_t* wc = wo + (long)ci * kh * kw;
                        for (int ky = 0; ky < kh; ++ky) {
                            const int iy = oy * sh - ph + ky * dh;
                            if (iy < 0 || iy >= h) continue;
                            for (int kx = 0; kx < kw; ++kx) {
                                const int ix = ox * sw - pw + kx * dw;
                                if (ix < 0 || ix >= w) continue;
                                sum += (int32_t)xc[(long)iy * w + ix] * (int32_t)wc[ky * kw + kx];
                            }
                        }
                    }
                    dst[(long)oy * ow + ox] = sum;
                }
        }
}

/* QuantizeX86.hpp:72-106 (packed) and QuantizeX86.cpp:25-45 (scalar); identical results for 0..3:
 * LeakyReLU packed = max(v,0) + slope*min(v,0): one addend is always zero, so one rounding. */
static inline float orc_act(float v, int act_type, float p0) {
    switch (act_type) {
        case ORC_ACT_RELU: return v > 0.f ? v : 0.f;
        case ORC_ACT_LRELU: return v > 0.f ? v : v * p0;
        case ORC_ACT_RELU6: {
            if (v < 0.f) v = 0.f;
            if (v > 6.f) v = 6.f;
            return v;
        }
        default: return v;
    }
}

void orc_dequantize(const int32_t* acc, int n, int c, int hw, const float* scale_in, int n_scale_in,
                    const float* bias, int n_bias, int act_type, float act_param0, float* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b)
        for (int q = 0; q < c; ++q) {
            const float s = n_scale_in == 1 ? scale_in[0] : scale_in[q];
            const float bq = n_bias == 0 ? 0.f : (n_bias == 1 ? bias[0] : bias[q]);
            const int32_t* src = acc + ((long)b * c + q) * hw;
            float* dst = out + ((long)b * c + q) * hw;
            for (long i = 0; i < hw; ++i) {
                float v = n_bias == 0 ? (float)src[i] * s : fmaf((float)src[i], s, bq);
                dst[i] = orc_act(v, act_type, act_param0);
            }
        }
}

void orc_requantize(const int32_t* acc, int n, int c, int hw, const float* scale_in, int n_scale_in,
                    const float* scale_out, int n_scale_out, const float* bias, int n_bias,
                    int act_type, float act_param0, int rounding, int8_t* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b)
        for (int q = 0; q < c; ++q) {
            const float s = n_scale_in == 1 ? scale_in[0] : scale_in[q];
            const float so = n_scale_out == 1 ? scale_out[0] : scale_out[q];
            const float bq = n_bias == 0 ? 0.f : (n_bias == 1 ? bias[0] : bias[q]);
            const int32_t* src = acc + ((long)b * c + q) * hw;
            int8_t* dst = out + ((long)b * c + q) * hw;
            for (long i = 0; i < hw; ++i) {
                float v = n_bias == 0 ? (float)src[i] * s : fmaf((float)src[i], s, bq);
                v = orc_act(v, act_type, act_param0);
                dst[i] = orc_float2int8(v * so, rounding);
            }
        }
}

int orc_conv_int8_forward(const orc_conv_desc* d, const int8_t* w_oihw, const float* bias,
                          const float* w_scales, const float* in_scales, int n_in_scales,
                          const float* out_scales, int n_out_scales,
                          const float* x_f32, const int8_t* x_s8, int n, int h, int w, int rounding,
                          int8_t* xq_out, int32_t* acc_out, float* y_f32, int8_t* y_s8) {
    const int oh = (h + 2 * d->ph - d->dh * (d->kh - 1) - 1) / d->sh + 1;
    const int ow = (w + 2 * d->pw - d->dw * (d->kw - 1) - 1) / d->sw + 1;
    const long in_elems = (long)n * d->cin * h * w, out_elems = (long)n * d->cout * oh * ow;
    int8_t* xq = NULL;
    const int8_t* xin = x_s8;
    if (x_f32) {
        xq = (int8_t*)malloc(in_elems > 0 ? in_elems : 1);
        if (!xq) return -100;
        orc_quantize(x_f32, n, d->cin, h, w, in_scales, n_in_scales, rounding, xq);
        xin = xq;
    }
    if (xq_out) memcpy(xq_out, xin, in_elems);
    int32_t* acc = acc_out ? acc_out : (int32_t*)malloc((out_elems > 0 ? out_elems : 1) * sizeof(int32_t));
    if (!acc) { free(xq); return -100; }
    orc_conv_s32(xin, n, d->cin, h, w, w_oihw, d->cout, d->kh, d->kw, d->sh, d->sw, d->ph, d->pw, d->dh, d->dw,
                 d->groups, acc);
    float* scale_in = (float*)malloc(sizeof(float) * (d->cout > 0 ? d->cout : 1));
    orc_scale_in(w_scales, d->cout, in_scales[0], scale_in);
    const int nb = d->bias_term ? d->cout : 0;
    if (d->int8_scale_term > 100) {
        if (y_s8)
            orc_requantize(acc, n, d->cout, oh * ow, scale_in, d->cout, out_scales, n_out_scales, bias, nb,
                           d->act_type, d->act_param0, rounding, y_s8);
    } else if (y_f32) {
        orc_dequantize(acc, n, d->cout, oh * ow, scale_in, d->cout, bias, nb, d->act_type, d->act_param0, y_f32);
    }
    free(scale_in);
    if (!acc_out) free(acc);
    free(xq);
    return 0;
}

/* ---- bilinear Upsample (fp32 glue between the convolutions of the detector graphs) ---- */
typedef struct { int i0, i1; float w0, w1; } orc_tap;

static orc_tap orc_axis_tap(int d, int in, int out, double user_scale, int packed_rule) {
    orc_tap t;
    if (packed_rule) { /* Tensor/TensorInterpolation.cpp:16-46 */
        const double scale = (double)in / out;
        float f = (float)((d + 0.5) * scale - 0.5);
        int s = (int)floor(f);
        f -= (float)s;
        if (s < 0) { s = 0; f = 0.f; }
        if (s >= in - 1) { s = in - 2; f = 1.f; }
        t.i0 = s; t.i1 = s + 1; t.w0 = 1.f - f; t.w1 = f;
        return t;
    }
    /* Tensor/UpSample.hpp:41-51,72-94,133-158 */
    if (out == in) { t.i0 = t.i1 = d; t.w0 = 1.f; t.w1 = 0.f; return t; }
    const float ratio = user_scale > 0. ? (float)(1.0 / user_scale) : (float)in / (float)out;
    float real = (float)((double)ratio * (d + 0.5) - 0.5);
    if (real < 0.f) real = 0.f;
    t.i0 = (int)real;
    t.i1 = t.i0 + (t.i0 < in - 1 ? 1 : 0);
    t.w1 = real - (float)t.i0;
    t.w0 = 1.f - t.w1;
    return t;
}

void orc_upsample_bilinear(const float* x, int n, int c, int h, int w, int oh, int ow, double scale_h, double scale_w,
                           int packed_rule, float* y) {
    const long planes = (long)n * c;
#pragma omp parallel for schedule(static)
    for (long p = 0; p < planes; ++p) {
        const float* xp = x + p * (long)h * w;
        float* yp = y + p * (long)oh * ow;
        for (int oy = 0; oy < oh; ++oy) {
            const orc_tap ty = orc_axis_tap(oy, h, oh, scale_h, packed_rule);
            for (int ox = 0; ox < ow; ++ox) {
                const orc_tap tx = orc_axis_tap(ox, w, ow, scale_w, packed_rule);
                const float a00 = xp[(long)ty.i0 * w + tx.i0], a01 = xp[(long)ty.i0 * w + tx.i1];
                const float a10 = xp[(long)ty.i1 * w + tx.i0], a11 = xp[(long)ty.i1 * w + tx.i1];
                float v;
                if (packed_rule) {
                    const float r0 = fmaf(a01, tx.w1, a00 * tx.w0), r1 = fmaf(a11, tx.w1, a10 * tx.w0);
                    v = fmaf(r1, ty.w1, r0 * ty.w0);
                } else {
                    const float r0 = fmaf(a00, tx.w0, a01 * tx.w1), r1 = fmaf(a10, tx.w0, a11 * tx.w1);
                    v = fmaf(r0, ty.w0, r1 * ty.w1);
                }
                yp[(long)oy * ow + ox] = v;
            }
        }
    }
}

/* Source index of the nearest resize along one axis. Packed blobs: ratio in/out in fp32, product truncated
 * (Tensor/TensorInterpolation.cpp:660-676). Plain blobs: copy when the sizes agree, index >> 1 when the size doubles,
 * else floor(d * (float)(1 / scale)) (Tensor/UpSampleKernel.cpp:41-60, Tensor/UpSample.hpp:30-51). */
static int orc_nearest_index(int d, int in, int out, double user_scale, int packed_rule) {
    int i;
    if (packed_rule) {
        const float ratio = (float)in / (float)out;
        i = (int)((float)d * ratio);
    } else {
        if (out == in) return d;
        if (out == 2 * in) return d >> 1;
        const float ratio = user_scale > 0. ? (float)(1.0 / user_scale) : (float)in / (float)out;
        i = (int)floorf((float)d * ratio);
    }
    return i < in - 1 ? i : in - 1;
}

void orc_upsample_nearest(const float* x, int n, int c, int h, int w, int oh, int ow, double scale_h, double scale_w,
                          int packed_rule, float* y) {
    const long planes = (long)n * c;
#pragma omp parallel for schedule(static)
    for (long p = 0; p < planes; ++p) {
        const float* xp = x + p * (long)h * w;
        float* yp = y + p * (long)oh * ow;
        for (int oy = 0; oy < oh; ++oy) {
            const int iy = orc_nearest_index(oy, h, oh, scale_h, packed_rule);
            for (int ox = 0; ox < ow; ++ox) yp[(long)oy * ow + ox] = xp[(long)iy * w + orc_nearest_index(ox, w, ow, scale_w, packed_rule)];
        }
    }
}

/* ---- detection decode of the NanoDet-Plus head ---- */
typedef struct { float x, y, w, h, prob; int label; int order; } orc_det;

static int orc_det_cmp(const void* a, const void* b) {
    const orc_det* p = (const orc_det*)a;
    const orc_det* q = (const orc_det*)b;
    if (p->prob != q->prob) return p->prob > q->prob ? -1 : 1;
    return p->order - q->order;
}

static float orc_intersection(const orc_det* a, const orc_det* b) { /* :192-206 */
    const float axmax = a->x + a->w, aymax = a->y + a->h, bxmax = b->x + b->w, bymax = b->y + b->h;
    if (a->x > bxmax || axmax < b->x || a->y > bymax || aymax < b->y) return 0.f;
    const float iw = fminf(axmax, bxmax) - fmaxf(a->x, b->x);
    const float ih = fminf(aymax, bymax) - fmaxf(a->y, b->y);
    return iw * ih;
}

int orc_nanodet_detect(const float* const* heads, const int* gh, const int* gw, const int* strides, int n_levels, int num_class,
                       int reg_bins, float prob_threshold, float nms_threshold, float* out, int max_det) {
    long cells = 0;
    for (int l = 0; l < n_levels; ++l) cells += (long)gh[l] * gw[l];
    orc_det* props = (orc_det*)malloc(sizeof(orc_det) * (size_t)(cells > 0 ? cells : 1));
    int n = 0;
    for (int l = 0; l < n_levels; ++l) { /* generate_proposals, :111-190 */
        const long plane = (long)gh[l] * gw[l];
        const float* pred = heads[l];
        for (int i = 0; i < gh[l]; ++i)
            for (int j = 0; j < gw[l]; ++j) {
                int label = -1;
                float score = -FLT_MAX;
                for (int k = 0; k < num_class; ++k) {
                    const float s = pred[k * plane + (long)i * gw[l] + j];
                    if (s > score) { label = k; score = s; }
                }
                score = 1.0f / (1.0f + expf(-score));
                if (!(score >= prob_threshold)) continue;
                float ltrb[4];
                for (int side = 0; side < 4; ++side) {
                    float v[64], m = -FLT_MAX, sum = 0.f, dis = 0.f;
                    for (int b = 0; b < reg_bins; ++b) {
                        v[b] = pred[(num_class + side * reg_bins + b) * plane + (long)i * gw[l] + j];
                        m = fmaxf(m, v[b]);
                    }
                    for (int b = 0; b < reg_bins; ++b) { v[b] = expf(v[b] - m); sum += v[b]; }
                    for (int b = 0; b < reg_bins; ++b) { v[b] /= sum; dis += (float)b * v[b]; }
                    ltrb[side] = dis * (float)strides[l];
                }
                const float cx = (float)(j * strides[l]), cy = (float)(i * strides[l]);
                const float x0 = cx - ltrb[0], y0 = cy - ltrb[1], x1 = cx + ltrb[2], y1 = cy + ltrb[3];
                orc_det d = {x0, y0, x1 - x0, y1 - y0, score, label, n};
                props[n++] = d;
            }
    }
    qsort(props, (size_t)n, sizeof(orc_det), orc_det_cmp);
    int* picked = (int*)malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
    int np = 0;
    for (int i = 0; i < n; ++i) { /* nms_sorted_bboxes, :208-243 */
        int keep = 1;
        const float area_i = props[i].w * props[i].h;
        for (int j = 0; j < np; ++j) {
            const orc_det* b = &props[picked[j]];
            const float inter = orc_intersection(&props[i], b);
            const float uni = area_i + b->w * b->h - inter;
            if (inter / uni > nms_threshold) keep = 0;
        }
        if (keep) picked[np++] = i;
    }
    for (int i = 0; i < np && i < max_det; ++i) {
        const orc_det* r = &props[picked[i]];
        float* o = out + 6 * i;
        o[0] = (float)(r->label + 1); o[1] = r->prob; o[2] = r->x; o[3] = r->y; o[4] = r->w; o[5] = r->h;
    }
    free(picked);
    free(props);
    return np;
}
