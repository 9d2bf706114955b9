"""GPU: the tensor-core depthwise 3x3 kernel (int8 NHWC input, stride 1 and 2) against the CPU checker and against the
CUDA-core kernel it replaces, bit for bit: channel counts with and without padding, ragged tiles, both output kinds, every
fused activation, and the shapes of the benchmark graphs."""
import numpy as np
import pytest

from support import ACT_LRELU, ACT_NONE, ACT_RELU, ACT_RELU6, ConvCase, nchw_to_nhwc_padded, nhwc_padded_to_nchw, run_port

pytestmark = pytest.mark.gpu

CASES = [
    # name, channels, stride, (n, h, w), int8_scale_term, activation
    ("c64_s1_f32", 64, 1, (1, 9, 11), 1, ACT_NONE),
    ("c58_s1_relu", 58, 1, (2, 40, 40), 101, ACT_RELU),
    ("c116_s1_none", 116, 1, (3, 20, 20), 101, ACT_NONE),
    ("c232_s1_lrelu", 232, 1, (2, 10, 10), 101, ACT_LRELU),
    ("c256_s1_relu6_f32", 256, 1, (1, 17, 23), 1, ACT_RELU6),
    ("c24_s2_none", 24, 2, (2, 80, 80), 101, ACT_NONE),
    ("c58_s2_relu", 58, 2, (2, 40, 40), 101, ACT_RELU),
    ("c116_s2_odd", 116, 2, (3, 21, 19), 101, ACT_NONE),
    ("c96_s2_f32", 96, 2, (1, 33, 47), 1, ACT_LRELU),
    ("c256_s2_big", 256, 2, (4, 56, 56), 101, ACT_RELU),
    ("c256_s1_many_tiles", 256, 1, (8, 56, 56), 101, ACT_RELU),
    ("c1_tiny", 40, 1, (1, 1, 1), 101, ACT_NONE),
]


@pytest.fixture(scope="module")
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


@pytest.mark.parametrize("dcase", CASES, ids=[c[0] for c in CASES])
def test_tensor_core_depthwise_bit_exact(ctx, dcase):
    from gpu_support import bits, make_layer
    from tensor_b200 import F32_NCHW, S8_NHWC, nhwc_channels
    name, c, stride, (n, h, w), term, act = dcase
    case = ConvCase(name, c, c, 3, stride, 1, groups=c, n=n, h=h, w=w, int8_scale_term=term, act_type=act, act_param0=0.1 if act == ACT_LRELU else 0.0,
                    w_std=0.1, s8_input=True, seed=500 + len(name)).make()
    want = run_port(case, 0, want_acc=False)["y"]
    layer = make_layer(ctx, case, 0)
    x = nchw_to_nhwc_padded(case.x_s8, nhwc_channels(c))
    x[..., c:] = -77  # padding channels of the input must not leak into real channels
    out_dtype = S8_NHWC if term > 100 else F32_NCHW
    got = {}
    for on in (2, 0):
        ctx.check(ctx.lib.ott_set_depthwise_tensor_cores(ctx.h, on))
        y = layer.forward_host(x, S8_NHWC, out_dtype)
        got[on] = nhwc_padded_to_nchw(y, c) if term > 100 else y
    ctx.check(ctx.lib.ott_set_depthwise_tensor_cores(ctx.h, 1))
    layer.close()
    assert np.array_equal(bits(got[0]), bits(want)), "CUDA-core kernel differs from the checker"
    assert np.array_equal(bits(got[2]), bits(want)), "tensor-core kernel differs from the checker"
