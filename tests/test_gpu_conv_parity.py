"""GPU parity: the CUDA path, called through the C-ABI, against the CPU checker on the same seeded
inputs and against the frozen reference outputs. Bit-exact for s32 accumulators, int8 and fp32 outputs
(tolerance: none)."""
import numpy as np
import pytest

from cases import small_cases
from support import GOLDEN_DIR, ACT_LRELU, ACT_RELU, ACT_RELU6, ConvCase, rounding_for, run_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


GOLD = np.load(GOLDEN_DIR / "conv_int8_small.npz")


@pytest.mark.parametrize("case,path", small_cases(), ids=[c.name for c, _ in small_cases()])
def test_small_case_bit_exact(ctx, case, path):
    from gpu_support import bits, run_gpu
    case.make()
    rounding = rounding_for(path)
    got = run_gpu(ctx, case, rounding)
    want = run_port(case, rounding)
    assert np.array_equal(got["acc"], want["acc"]), f"s32 accumulators differ (kernel kind {got['kind']})"
    assert not got["acc_pad"].any(), "padding channels of the accumulators must be zero"
    assert np.array_equal(bits(got["y"]), bits(want["y"])), f"final output differs (kernel kind {got['kind']})"
    assert np.array_equal(bits(got["y"]), bits(GOLD[case.name + "/y"])), "differs from the frozen reference output"
    if case.requant:
        assert not got["y_pad"].any(), "padding channels of the int8 output must be zero"


def test_kernel_selection(ctx):
    from gpu_support import make_layer
    from tensor_b200 import KERNEL_DENSE_DIRECT, KERNEL_DENSE_UMMA, KERNEL_DEPTHWISE
    expect = {"dw3x3s1_256_relu_s8": KERNEL_DEPTHWISE, "pw_64_256_relu6_s8": KERNEL_DENSE_UMMA,
              "dense3x3_64_f32": KERNEL_DENSE_UMMA, "stem_3_24_s2_f32": KERNEL_DENSE_DIRECT, "dense3x3_s2": KERNEL_DENSE_UMMA,
              "pw_512_1024_relu6_s8": KERNEL_DENSE_UMMA, "pw_464_1024": KERNEL_DENSE_UMMA}
    for case, _ in small_cases():
        if case.name in expect:
            case.make()
            layer = make_layer(ctx, case, 0)
            assert layer.kernel_kind == expect[case.name], case.name
            layer.close()


def test_batched_equals_single_images(ctx):
    """The reference is batch-1; a batched GPU call must give each image what a single-image call gives."""
    from gpu_support import bits, run_gpu
    case = ConvCase("batch", 64, 128, 1, n=5, h=9, w=13, int8_scale_term=101, act_type=ACT_RELU, seed=90).make()
    whole = run_gpu(ctx, case, 0, want_acc=False)["y"]
    for i in range(case.n):
        one = ConvCase("one", 64, 128, 1, n=1, h=9, w=13, int8_scale_term=101, act_type=ACT_RELU, seed=90).make()
        one.x_f32 = np.ascontiguousarray(case.x_f32[i:i + 1])
        one.in_scales, one.out_scales = case.in_scales, case.out_scales
        assert np.array_equal(bits(run_gpu(ctx, one, 0, want_acc=False)["y"]), bits(whole[i:i + 1]))


@pytest.mark.parametrize("name,kw", [
    ("many_tiles_pw", dict(cin=64, cout=256, k=1, n=6, h=56, w=56, int8_scale_term=101, act_type=ACT_RELU6)),
    ("many_tiles_3x3", dict(cin=64, cout=64, k=3, pad=1, n=4, h=56, w=56, int8_scale_term=2)),
    ("many_tiles_dw", dict(cin=256, cout=256, k=3, pad=1, groups=256, n=4, h=56, w=56, int8_scale_term=101, act_type=ACT_RELU, w_std=0.1)),
    ("dw_tiles_xy_f32in", dict(cin=40, cout=40, k=3, pad=1, groups=40, n=2, h=37, w=75, int8_scale_term=101, act_type=ACT_RELU, w_std=0.1)),
    ("dw_tiles_xy_s8in", dict(cin=72, cout=72, k=3, pad=1, groups=72, n=2, h=30, w=70, int8_scale_term=101, act_type=ACT_RELU6, w_std=0.1, s8_input=True)),
    ("dw_s2_tiles_f32out", dict(cin=48, cout=48, k=3, stride=2, pad=1, groups=48, n=1, h=45, w=83, int8_scale_term=1, w_std=0.1)),
    ("dw5_s1_tiles", dict(cin=96, cout=96, k=5, pad=2, groups=96, n=2, h=40, w=40, int8_scale_term=101, act_type=ACT_LRELU, act_param0=0.1, w_std=0.1, s8_input=True)),
    ("dw5_s2_tiles_w_odd", dict(cin=32, cout=32, k=5, stride=2, pad=2, groups=32, n=1, h=41, w=77, int8_scale_term=101, w_std=0.1)),
    ("dw_nopad", dict(cin=32, cout=32, k=3, pad=0, groups=32, n=1, h=20, w=24, int8_scale_term=101, act_type=ACT_RELU, w_std=0.1)),
    ("stem_odd_s2", dict(cin=3, cout=24, k=3, stride=2, pad=1, n=2, h=45, w=71, int8_scale_term=2, act_type=ACT_RELU, x_lo=0.0)),
    ("stem_s1_lrelu_s8", dict(cin=3, cout=16, k=3, stride=1, pad=1, n=2, h=33, w=40, int8_scale_term=101, act_type=ACT_LRELU, act_param0=0.1, x_lo=0.0)),
    ("stem_tiles", dict(cin=3, cout=24, k=3, stride=2, pad=1, n=3, h=96, w=160, int8_scale_term=2, act_type=ACT_RELU, x_lo=0.0)),
    # k x k dense layers read one halo tile per pixel tile through shifted operand views: every swizzle width, several
    # channel blocks, ragged tiles in both directions, no padding / wide padding, 5x5
    ("halo_3x3_c128", dict(cin=128, cout=128, k=3, pad=1, n=2, h=23, w=19, int8_scale_term=101, act_type=ACT_RELU, s8_input=True)),
    ("halo_3x3_c160_two_blocks", dict(cin=160, cout=96, k=3, pad=1, n=2, h=17, w=30, int8_scale_term=2)),
    ("halo_3x3_c32_nopad", dict(cin=32, cout=32, k=3, pad=0, n=2, h=21, w=12, int8_scale_term=2, act_type=ACT_LRELU, act_param0=0.1)),
    ("halo_3x3_c64_pad2", dict(cin=64, cout=48, k=3, pad=2, n=1, h=9, w=9, int8_scale_term=101, s8_input=True)),
    ("halo_5x5_c32", dict(cin=32, cout=64, k=5, pad=2, n=2, h=20, w=20, int8_scale_term=101, act_type=ACT_RELU6)),
    ("halo_3x1_c64", dict(cin=64, cout=64, k=3, kw=1, pad=0, n=2, h=19, w=11, int8_scale_term=2)),
    ("halo_1x3_c64", dict(cin=64, cout=32, k=1, kw=3, pad=0, n=2, h=10, w=21, int8_scale_term=101, act_type=ACT_RELU, s8_input=True)),
    ("dilated_3x3_c64_per_tap_boxes", dict(cin=64, cout=64, k=3, pad=2, dil=2, n=2, h=18, w=15, int8_scale_term=2, act_type=ACT_RELU)),
    # strided dense layers on the tensor cores: one TMA box per filter tap that takes every second (third) pixel
    ("strided_3x3_s2_c64_128", dict(cin=64, cout=128, k=3, stride=2, pad=1, n=3, h=56, w=56, int8_scale_term=101, act_type=ACT_RELU, s8_input=True)),
    ("strided_3x3_s2_odd_f32", dict(cin=32, cout=48, k=3, stride=2, pad=1, n=2, h=37, w=45, int8_scale_term=2)),
    ("strided_1x1_s2", dict(cin=64, cout=96, k=1, stride=2, pad=0, n=2, h=28, w=30, int8_scale_term=101, act_type=ACT_RELU6)),
    ("strided_5x5_s2_c32", dict(cin=32, cout=32, k=5, stride=2, pad=2, n=2, h=31, w=29, int8_scale_term=2, act_type=ACT_LRELU, act_param0=0.1)),
    ("strided_3x3_s3_nopad", dict(cin=48, cout=64, k=3, stride=3, pad=0, n=2, h=40, w=33, int8_scale_term=101, act_type=ACT_RELU, s8_input=True)),
    ("strided_3x3_s2_wide_rows", dict(cin=32, cout=32, k=3, stride=2, pad=1, n=1, h=6, w=300, int8_scale_term=2)),
    ("two_n_tiles", dict(cin=256, cout=512, k=1, n=3, h=28, w=28, int8_scale_term=101, act_type=ACT_RELU6)),
    ("four_n_tiles", dict(cin=512, cout=1024, k=1, n=2, h=14, w=14, int8_scale_term=101, act_type=ACT_RELU6)),
])
def test_medium_case_bit_exact(ctx, name, kw):
    """More pixel tiles than SMs, several weight panels: exercises the persistent loop and the pipelines."""
    from gpu_support import bits, run_gpu
    case = ConvCase(name, kw.pop("cin"), kw.pop("cout"), kw.pop("k"), kw.pop("stride", 1), kw.pop("pad", 0), seed=91, **kw).make()
    got = run_gpu(ctx, case, 0)
    want = run_port(case, 0)
    assert np.array_equal(got["acc"], want["acc"])
    assert np.array_equal(bits(got["y"]), bits(want["y"]))
