"""The seeded parity cases shared by the CPU and GPU tests.

SMALL_CASES are sized so every checker finishes in well under a second; they cover the shapes the
benchmark configurations use (scaled down spatially), the edge shapes (channel counts that need
padding, odd spatial sizes, 5x5, stride 2, no bias, int8 input, every fused activation) and both
output kinds. `path` says which reference code path is the checker of record for the case:
"packed" (use_packing_layout=true, the default; valid when Cin%8==0 and Cout%4==0, and for the 3->24
stem), "unpacked" for other dense widths, "port" where the reference itself cannot run the shape
(depthwise with C%8 != 0 corrupts its heap): there the s32 accumulators come from the restatement and
the epilogue is the reference's own requantize/dequantize function, packed when C%4==0, else unpacked
(the unpacked fp32 epilogue additionally needs H*W%4==0 to dodge a tail defect of the reference).
"""
from support import ACT_LRELU, ACT_NONE, ACT_RELU, ACT_RELU6, ConvCase


def small_cases():
    C = ConvCase
    return [
        # config 1 scaled down: dense 3x3 s1 p1 64->64, fp32 in/out
        (C("dense3x3_64_f32", 64, 64, 3, 1, 1, n=2, h=14, w=14, int8_scale_term=2, seed=1), "packed"),
        # config 2 scaled down: depthwise 3x3 s1/s2, ReLU, int8 out
        (C("dw3x3s1_256_relu_s8", 256, 256, 3, 1, 1, groups=256, n=2, h=14, w=14, int8_scale_term=101, act_type=ACT_RELU, w_std=0.1, seed=2), "packed"),
        (C("dw3x3s2_256_relu_s8", 256, 256, 3, 2, 1, groups=256, n=2, h=14, w=14, int8_scale_term=101, act_type=ACT_RELU, w_std=0.1, seed=3), "packed"),
        # config 3 scaled down: pointwise, ReLU6, int8 out
        (C("pw_64_256_relu6_s8", 64, 256, 1, n=2, h=14, w=14, int8_scale_term=101, act_type=ACT_RELU6, seed=4), "packed"),
        (C("pw_256_512_relu6_s8", 256, 512, 1, n=1, h=7, w=7, int8_scale_term=101, act_type=ACT_RELU6, seed=5), "packed"),
        (C("pw_512_1024_relu6_s8", 512, 1024, 1, n=1, h=4, w=4, int8_scale_term=101, act_type=ACT_RELU6, seed=6), "packed"),
        # activations and output kinds
        (C("pw_lrelu_s8", 64, 128, 1, n=1, h=7, w=9, int8_scale_term=101, act_type=ACT_LRELU, act_param0=0.1, seed=7), "packed"),
        (C("pw_lrelu_f32", 64, 128, 1, n=1, h=8, w=8, int8_scale_term=2, act_type=ACT_LRELU, act_param0=0.1, seed=8), "packed"),
        (C("pw_relu_f32", 32, 64, 1, n=1, h=8, w=8, int8_scale_term=2, act_type=ACT_RELU, seed=9), "packed"),
        (C("pw_relu6_f32", 32, 64, 1, n=1, h=8, w=8, int8_scale_term=2, act_type=ACT_RELU6, w_std=0.5, seed=10), "packed"),
        (C("pw_nobias_s8", 64, 64, 1, n=1, h=12, w=12, int8_scale_term=102, bias_term=0, seed=11), "packed"),
        (C("pw_nobias_f32", 64, 64, 1, n=1, h=12, w=12, int8_scale_term=2, bias_term=0, seed=12), "packed"),
        # int8 activations arriving from a requantizing producer
        (C("dense3x3_s8in_relu_s8", 64, 64, 3, 1, 1, n=1, h=12, w=12, int8_scale_term=102, s8_input=True, act_type=ACT_RELU, seed=13), "packed"),
        (C("dw3x3_s8in_f32", 64, 64, 3, 1, 1, groups=64, n=1, h=9, w=11, int8_scale_term=1, s8_input=True, w_std=0.1, seed=14), "packed"),
        # 5x5 depthwise (detector neck/head), stride 1 and 2
        (C("dw5x5s1_96", 96, 96, 5, 1, 2, groups=96, n=1, h=20, w=20, int8_scale_term=1, w_std=0.1, seed=15), "packed"),
        (C("dw5x5s2_96_lrelu_s8", 96, 96, 5, 2, 2, groups=96, n=2, h=20, w=20, int8_scale_term=101, act_type=ACT_LRELU, act_param0=0.1, w_std=0.1, seed=16), "packed"),
        # stem: 3 -> 24, 3x3 s2, fp32 image in [0,1]
        (C("stem_3_24_s2_f32", 3, 24, 3, 2, 1, n=2, h=32, w=32, int8_scale_term=2, x_lo=0.0, seed=17), "packed"),
        (C("stem_3_24_s2_relu_s8", 3, 24, 3, 2, 1, n=1, h=32, w=32, int8_scale_term=101, act_type=ACT_RELU, x_lo=0.0, seed=18), "packed"),
        # channel counts of ShuffleNetV2-1.0x that need padding on the GPU
        (C("pw_24_58", 24, 58, 1, n=1, h=10, w=10, int8_scale_term=101, act_type=ACT_RELU, seed=19), "packed_pack8to1"),
        (C("pw_58_58_unpacked", 58, 58, 1, n=1, h=20, w=20, int8_scale_term=101, act_type=ACT_RELU, seed=20), "unpacked"),
        (C("pw_116_116_unpacked_f32", 116, 116, 1, n=1, h=10, w=10, int8_scale_term=2, seed=21), "unpacked"),
        (C("pw_232_232", 232, 232, 1, n=1, h=6, w=6, int8_scale_term=101, act_type=ACT_RELU, seed=22), "packed"),
        (C("pw_464_1024", 464, 1024, 1, n=1, h=3, w=5, int8_scale_term=2, act_type=ACT_RELU, seed=23), "packed"),
        (C("dw3x3s2_58_port", 58, 58, 3, 2, 1, groups=58, n=1, h=16, w=16, int8_scale_term=101, w_std=0.1, seed=24), "port_unpacked_epilogue"),
        (C("dw3x3s1_116_port_f32", 116, 116, 3, 1, 1, groups=116, n=1, h=7, w=7, int8_scale_term=1, w_std=0.1, seed=25), "port_packed_epilogue"),
        # odd spatial sizes / non-square / larger dense kernels
        (C("dense3x3_odd", 32, 48, 3, 1, 1, n=3, h=5, w=7, int8_scale_term=101, act_type=ACT_RELU, seed=26), "packed"),
        (C("dense3x3_s2", 32, 64, 3, 2, 1, n=1, h=9, w=9, int8_scale_term=101, act_type=ACT_RELU6, seed=27), "packed"),
        (C("dense3x3_nopad", 16, 32, 3, 1, 0, n=1, h=6, w=6, int8_scale_term=2, seed=28), "packed"),
        (C("dense5x5", 16, 16, 5, 1, 2, n=1, h=8, w=8, int8_scale_term=2, seed=29), "packed"),
        (C("pw_1x1_spatial1", 128, 64, 1, n=4, h=1, w=1, int8_scale_term=101, act_type=ACT_RELU, seed=30), "packed"),
        (C("pw_96_112_head", 96, 112, 1, n=1, h=10, w=10, int8_scale_term=2, seed=31), "packed"),
    ]
