"""GPU: the fused pair kernel (depthwise 3x3 stride 1 / 2 -> 1x1 convolution in one launch, ott_dwpw_*) against the two layers
run one after the other through the CPU checker, bit for bit: int8 / fp32 / mixed output, the channel counts of
ShuffleNetV2-1.0x (24, 58, 116, 232) and others, every buffering mode of the kernel (two CTAs per SM, one CTA with double
buffers, single buffers for the widest layers; one or several input chunks per tile), ragged tiles, and the benchmarked
geometry with many more tiles than resident CTAs."""
import copy

import numpy as np
import pytest

from support import ACT_LRELU, ACT_NONE, ACT_RELU, ACT_RELU6, ConvCase, nchw_to_nhwc_padded, nhwc_padded_to_nchw, run_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


def _layer(ctx, case, **kw):
    from tensor_b200 import ConvInt8
    return ConvInt8(ctx, cin=case.cin, cout=case.cout, kh=case.k, kw=case.k, sh=case.stride, sw=case.stride, ph=case.pad, pw=case.pad, groups=case.groups,
                    bias_term=1, int8_scale_term=case.int8_scale_term, act_type=case.act_type, act_param0=case.act_param0, rounding=0, weight=case.weight,
                    bias=case.bias, w_scales=case.w_scales, in_scales=case.in_scales, out_scales=case.out_scales if case.requant else None, **kw)


def _rescale(case):
    """Output scale of a requantizing layer from the values it actually sees: 127 / max |fp32 output|."""
    if not case.requant:
        return
    probe = copy.copy(case)
    probe.int8_scale_term = case.int8_scale_term - 100
    y = run_port(probe, 0, want_acc=False)["y"]
    case.out_scales = np.full_like(case.out_scales, np.float32(127.0) / np.float32(max(float(np.abs(y).max()), 1e-6)))


def _pair(cm, cout, stride, n, h, w, act, term2, seed, act_param0=0.0):
    """Two seeded layers and the checker's result of running them one after the other on a seeded int8 input."""
    dw = ConvCase("p_dw", cm, cm, 3, stride, 1, groups=cm, n=n, h=h, w=w, int8_scale_term=101, act_type=ACT_NONE, w_std=0.1, s8_input=True, seed=seed).make()
    _rescale(dw)
    y1 = run_port(dw, 0, want_acc=False)["y"]
    oh, ow = y1.shape[2], y1.shape[3]
    pw = ConvCase("p_pw", cm, cout, 1, n=n, h=oh, w=ow, int8_scale_term=term2, act_type=act, act_param0=act_param0, s8_input=True, seed=seed + 1).make()
    pw.x_s8 = y1
    _rescale(pw)
    y2 = run_port(pw, 0, want_acc=False)["y"]
    assert np.abs(y1).max() > 20, "degenerate test data"
    return dw, pw, y2


PAIR_CASES = [
    # name, channels, cout, stride, (n, h, w), activation, int8_scale_term of the 1x1 layer
    ("c58_s1", 58, 58, 1, (2, 12, 12), ACT_RELU, 101),
    ("c116_s1_ragged_f32", 116, 116, 1, (3, 13, 21), ACT_RELU, 2),
    ("c24_s2", 24, 58, 2, (2, 20, 20), ACT_RELU, 101),
    ("c58_s2_ragged", 58, 58, 2, (2, 21, 17), ACT_RELU, 2),
    ("c116_s2", 116, 116, 2, (2, 40, 40), ACT_RELU, 101),
    ("c232_s1", 232, 232, 1, (3, 10, 10), ACT_RELU, 2),
    ("c232_s2", 232, 232, 2, (2, 20, 20), ACT_RELU, 101),
    ("c64_lrelu", 64, 96, 1, (1, 17, 9), ACT_LRELU, 101),
    ("c40_relu6_small", 40, 24, 1, (2, 5, 7), ACT_RELU6, 102),
    ("c176_none_f32", 176, 112, 1, (1, 20, 20), ACT_NONE, 2),
    ("c256_s1_wide_out", 256, 256, 1, (1, 9, 33), ACT_RELU, 101),
    # the benchmarked geometry: ShuffleNetV2-1.0x at 320x320, more tiles than resident CTAs
    ("stage2_hw40", 58, 58, 1, (32, 40, 40), ACT_RELU, 2),
    ("stage3_hw20", 116, 116, 1, (48, 20, 20), ACT_RELU, 2),
    ("stage4_hw10", 232, 232, 1, (96, 10, 10), ACT_RELU, 2),
    ("stage2_entry_s2_hw80", 58, 58, 2, (12, 80, 80), ACT_RELU, 2),
    ("stage3_entry_s2_hw40", 116, 116, 2, (24, 40, 40), ACT_RELU, 2),
]


@pytest.mark.parametrize("pcase", PAIR_CASES, ids=[c[0] for c in PAIR_CASES])
def test_pair_plain_input_bit_exact(ctx, pcase):
    from gpu_support import bits
    from tensor_b200 import DwPwInt8, F32_NCHW, S8_NHWC, nhwc_channels
    name, cm, cout, stride, (n, h, w), act, term2 = pcase
    dw, pw, want = _pair(cm, cout, stride, n, h, w, act, term2, seed=2000 + len(name) + cm, act_param0=0.1 if act == ACT_LRELU else 0.0)
    ld, lp = _layer(ctx, dw), _layer(ctx, pw)
    pair = DwPwInt8(ctx, ld, lp)
    x = nchw_to_nhwc_padded(dw.x_s8, nhwc_channels(cm))
    x[..., cm:] = 33  # whatever lies in the padding channels must not matter
    xd = ctx.to_device(x)
    out_dtype = S8_NHWC if term2 > 100 else F32_NCHW
    oh, ow = want.shape[2], want.shape[3]
    out = lp.out_array(n, oh, ow, out_dtype)
    od = ctx.malloc(out.nbytes)
    ctx.memset(od, 0x5A, out.nbytes)
    try:
        for _ in range(2):
            pair.forward_io(n, h, w, od, out_dtype, in_dev=xd)
        got = ctx.to_host(od, out.shape, out.dtype)
        if term2 > 100:
            assert not got[..., cout:].any()
            got = nhwc_padded_to_nchw(got, cout)
        assert np.array_equal(bits(got), bits(want))
    finally:
        ctx.free(xd)
        ctx.free(od)
        pair.close()
        ld.close()
        lp.close()


def test_pair_mixed_output(ctx):
    """The output form the graph uses: per-channel-scaled int8 plus fp32 planes for some channels."""
    from gpu_support import bits
    from tensor_b200 import DwPwInt8, S8_NHWC, nhwc_channels
    rng = np.random.default_rng(6)
    n, h, w, c = 5, 40, 40, 58
    dw, pw, _ = _pair(c, c, 1, n, h, w, ACT_RELU, 101, seed=99)
    f32_channels = sorted(rng.choice(c, size=c // 3, replace=False).tolist())
    scales = np.full(c, pw.out_scales[0], np.float32) * rng.uniform(0.5, 1.5, c).astype(np.float32)
    scales[f32_channels] = 0.0
    pw.out_scales = scales
    want_s8 = run_port(pw, 0, want_acc=False)["y"]
    fcase = copy.copy(pw)
    fcase.int8_scale_term, fcase.out_scales = 1, np.zeros(1, np.float32)
    want_f32 = run_port(fcase, 0, want_acc=False)["y"]
    ld, lp = _layer(ctx, dw), _layer(ctx, pw)
    pair = DwPwInt8(ctx, ld, lp)
    xd = ctx.to_device(nchw_to_nhwc_padded(dw.x_s8, nhwc_channels(c)))
    out = lp.out_array(n, h, w, S8_NHWC)
    od = ctx.malloc(out.nbytes)
    side = np.full((n, c, h, w), -12345.0, np.float32)
    sd = ctx.to_device(side)
    try:
        pair.forward_io(n, h, w, od, S8_NHWC, in_dev=xd, out_f32_dev=sd, f32_channels=f32_channels)
        got_s8 = nhwc_padded_to_nchw(ctx.to_host(od, out.shape, out.dtype), c)
        got_f32 = ctx.to_host(sd, side.shape, side.dtype)
        assert np.array_equal(got_s8, want_s8)
        assert np.array_equal(bits(got_f32[:, f32_channels]), bits(want_f32[:, f32_channels]))
        others = [ch for ch in range(c) if ch not in set(f32_channels)]
        assert (got_f32[:, others] == -12345.0).all()
    finally:
        for p in (xd, od, sd):
            ctx.free(p)
        pair.close()
        ld.close()
        lp.close()


def test_pair_refuses_what_it_cannot_fuse(ctx):
    from tensor_b200 import DwPwInt8, OtterB200Error
    dw, pw, _ = _pair(64, 64, 1, 1, 8, 8, ACT_RELU, 101, seed=3)
    wide_dw, wide_pw, _ = _pair(320, 64, 1, 1, 8, 8, ACT_RELU, 101, seed=4)
    other_dw, other_pw, _ = _pair(32, 64, 1, 1, 8, 8, ACT_RELU, 101, seed=5)
    layers = [_layer(ctx, c) for c in (dw, pw, wide_dw, wide_pw, other_pw)]
    ld, lp, wd, wp, op = layers
    with pytest.raises(OtterB200Error):  # layers in the wrong order
        DwPwInt8(ctx, lp, ld)
    with pytest.raises(OtterB200Error):  # more depthwise channels than tensor memory holds
        DwPwInt8(ctx, wd, wp)
    with pytest.raises(OtterB200Error):  # channel counts do not chain
        DwPwInt8(ctx, ld, op)
    for l in layers:
        l.close()
