/* CPU restatement of the reference's int8 convolution path — TEST INFRASTRUCTURE ONLY.
 *
 * Only the parity tests, the smoke check and the bench's CPU-baseline leg may load this.
 * The GPU library never links or calls it, and has no CPU path of its own.
 *
 * Parity status: PINNED. Every function here is checked bit-for-bit against the reference's own
 * compiled code (oracle/_ref/libotter_ref.so, built by oracle/Makefile from the reference sources)
 * by tests/test_oracle_vs_reference.py, and against the frozen outputs of that library under
 * tests/golden/ by tests/test_oracle_golden.py. The reference ships no golden vectors or
 * known-answer tests for this path.
 */
#ifndef OTTER_INT8_ORACLE_H
#define OTTER_INT8_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* How a float becomes an int8.
 * ORC_ROUND_ADD_HALF_TRUNC: v + copysign(0.5, v) in fp32, truncate, clamp to [-127,127]
 *     = float2int8_sse, the packed (default) x86 path: Tensor/VecIntrinsic.hpp:71-161.
 * ORC_ROUND_HALF_AWAY: round() half away from zero, clamp to [-127,127]
 *     = scalar float2int8, the unpacked x86 path: Tensor/QuantizeX86.cpp:18-23
 *     (also aarch64 vcvtaq: Tensor/QuantizeNeon.hpp:27-29).
 * They differ only at |v| = 0.49999997f. */
enum { ORC_ROUND_ADD_HALF_TRUNC = 0, ORC_ROUND_HALF_AWAY = 1 };

/* activation codes of ConvolutionLayer::parse_param, Tensor/ConvolutionLayer.cpp:121-131 */
enum { ORC_ACT_NONE = 0, ORC_ACT_RELU = 1, ORC_ACT_LRELU = 2, ORC_ACT_RELU6 = 3 };

typedef struct {
    int cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups;
    int bias_term;
    int int8_scale_term; /* 1,2: fp32 output ; 101,102: int8 output */
    int act_type;
    float act_param0;    /* LeakyReLU slope */
} orc_conv_desc;

int8_t orc_float2int8(float v, int rounding);

/* scale_in[p] = w_scale[p]==0 ? 0 : 1/(in_scale0 * w_scale[p])  — ConvolutionLayer.cpp:667-679 */
void orc_scale_in(const float* w_scales, int cout, float in_scale0, float* scale_in);

/* fp32 NCHW -> int8 NCHW ; scale per tensor (n_scales==1) or per channel — QuantizeX86.cpp:47-644 */
void orc_quantize(const float* x, int n, int c, int h, int w, const float* scales, int n_scales,
                  int rounding, int8_t* out);

/* exact s32 accumulators, NCHW, groups supported (dense: groups=1, depthwise: groups=cin=cout),
 * zero padding, stride, dilation — the 7-loop statement Tensor/ConvolutionMM2D.cpp:553-649;
 * same sums as ConvolutionMM2DInt8X86Pack.cpp:1656-2223 and DepthwiseConvKernelInt8X86Pack.cpp:19-119. */
void orc_conv_s32(const int8_t* x, int n, int cin, int h, int w, const int8_t* w_oihw, int cout,
                  int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups, int32_t* acc);

/* y = fma((float)acc, scale_in[c], bias[c]) (no bias: (float)acc*scale_in[c]) — QuantizeX86.cpp:646-1161
 * as compiled with the reference's -Ofast -mfma flags; then the stand-alone activation layer
 * ConvolutionLayer.cpp:841-843 (ReluLayer / LReluLayer / Relu6Layer). */
void orc_dequantize(const int32_t* acc, int n, int c, int hw, const float* scale_in, int n_scale_in,
                    const float* bias, int n_bias, int act_type, float act_param0, float* out);

/* q = float2int8(act(fma(acc, scale_in[c], bias[c])) * scale_out[c or 0]) — QuantizeX86.cpp:1163-2125,
 * activation QuantizeX86.hpp:72-106 / QuantizeX86.cpp:25-45. */
void orc_requantize(const int32_t* acc, int n, int c, int hw, const float* scale_in, int n_scale_in,
                    const float* scale_out, int n_scale_out, const float* bias, int n_bias,
                    int act_type, float act_param0, int rounding, int8_t* out);

/* The whole ConvolutionLayer::forward_int8 (ConvolutionLayer.cpp:754-847) on NCHW buffers.
 * Exactly one of x_f32 / x_s8 is non-NULL. Optional outputs may be NULL. Returns 0. */
int orc_conv_int8_forward(const orc_conv_desc* d, const int8_t* w_oihw, const float* bias,
                          const float* w_scales, const float* in_scales, int n_in_scales,
                          const float* out_scales, int n_out_scales,
                          const float* x_f32, const int8_t* x_s8, int n, int h, int w, int rounding,
                          int8_t* xq_out, int32_t* acc_out, float* y_f32, int8_t* y_s8);

/* UpsampleLayer::forward for upsample_mode = bilinear, align_corner = false (Tensor/UpsampleLayer.cpp:113-131), fp32 NCHW.
 * packed_rule 1: the reference's resize of packed blobs (channels % 4 == 0 under use_packing_layout): coefficients
 *   of linear_coeffs (Tensor/TensorInterpolation.cpp:16-46), rows = fma(S1, a1, S0 * a0), D = fma(rows1, b1, rows0 * b0)
 *   (:199-207,:251-259).
 * packed_rule 0: its resize of plain blobs: coefficients of compute_source_index_and_lambda (Tensor/UpSample.hpp:133-158,
 *   scale from compute_scales_value :41-51), t0 * w0 + t1 * w1 per axis (Tensor/UpSampleKernel.cpp:125-139), which the
 *   reference build (-Ofast -mfma) evaluates as fma(t0, w0, t1 * w1).
 * scale_h / scale_w: the layer's scale factors (used by rule 0 only; <= 0: in / out). */
void orc_upsample_bilinear(const float* x, int n, int c, int h, int w, int oh, int ow, double scale_h, double scale_w,
                           int packed_rule, float* y);

/* UpsampleLayer::forward for upsample_mode = nearest (Tensor/UpsampleLayer.cpp:113-131 -> otter::Interpolate): a copy of
 * the source pixel whose index the reference's two rules give (packed_rule as above). */
void orc_upsample_nearest(const float* x, int n, int c, int h, int w, int oh, int ow, double scale_h, double scale_w,
                          int packed_rule, float* y);

/* NanodetPlusDetectionOutputLayer::forward for one image (Tensor/NanodetPlusDetectionOutputLayer.cpp:65-260): per pyramid
 * level and grid cell the best of num_class logits, its sigmoid against prob_threshold, a softmax over the reg_bins
 * distance bins of each box side, the box; then all proposals sorted by score, greedy NMS. heads[l] is fp32
 * [num_class + 4*reg_bins][gh[l]][gw[l]]. out receives up to max_det rows {label + 1, score, x, y, width, height};
 * returns the number of detections kept (before truncation to max_det).
 * Floating point: exp is the C library's expf, as in the reference build; ties in the sort (equal scores) are broken by
 * proposal order (level, row, column), where the reference's quicksort leaves them unspecified. */
int orc_nanodet_detect(const float* const* heads, const int* gh, const int* gw, const int* strides, int n_levels, int num_class,
                       int reg_bins, float prob_threshold, float nms_threshold, float* out, int max_det);

int orc_max_threads(void);
void orc_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
