"""GPU: the fused unit kernel (1x1 convolution -> depthwise 3x3 -> 1x1 convolution in one launch, ott_unit_*) against the
three layers run one after the other through the CPU checker, bit for bit: plain and gathered input, int8 / fp32 / mixed
output, the channel counts of ShuffleNetV2-1.0x (58, 116) and others, ragged tiles, and the benchmarked geometry."""
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
    return ConvInt8(ctx, cin=case.cin, cout=case.cout, kh=case.k, kw=case.k, sh=1, sw=1, ph=case.pad, pw=case.pad, groups=case.groups, bias_term=1,
                    int8_scale_term=case.int8_scale_term, act_type=case.act_type, act_param0=case.act_param0, rounding=0, weight=case.weight,
                    bias=case.bias, w_scales=case.w_scales, in_scales=case.in_scales, out_scales=case.out_scales if case.requant else None, **kw)


def _rescale(case):
    """Output scale of a requantizing layer from the values it actually sees: 127 / max |fp32 output|."""
    if not case.requant:
        return
    probe = copy.copy(case)
    probe.int8_scale_term = case.int8_scale_term - 100
    y = run_port(probe, 0, want_acc=False)["y"]
    case.out_scales = np.full_like(case.out_scales, np.float32(127.0) / np.float32(max(float(np.abs(y).max()), 1e-6)))


def _chain(cin, cm, cout, n, h, w, act, term2, seed, act_param0=0.0):
    """Three seeded layers and the checker's result of running them one after the other on a seeded int8 input."""
    pw1 = ConvCase("u_pw1", cin, cm, 1, n=n, h=h, w=w, int8_scale_term=102, act_type=act, act_param0=act_param0, s8_input=True, seed=seed).make()
    y1 = run_port(pw1, 0, want_acc=False)["y"]
    dw = ConvCase("u_dw", cm, cm, 3, 1, 1, groups=cm, n=n, h=h, w=w, int8_scale_term=101, act_type=ACT_NONE, w_std=0.1, s8_input=True, seed=seed + 1).make()
    dw.x_s8 = y1
    _rescale(dw)
    y2 = run_port(dw, 0, want_acc=False)["y"]
    pw2 = ConvCase("u_pw2", cm, cout, 1, n=n, h=h, w=w, int8_scale_term=term2, act_type=act, act_param0=act_param0, s8_input=True, seed=seed + 2).make()
    pw2.x_s8 = y2
    _rescale(pw2)
    y3 = run_port(pw2, 0, want_acc=False)["y"]
    assert np.abs(y1).max() > 20 and np.abs(y2).max() > 20, "degenerate test data"
    return pw1, dw, pw2, y3


UNIT_CASES = [
    # name, cin, cm, cout, (n, h, w), activation, int8_scale_term of the last layer
    ("c58_hw12", 58, 58, 58, (2, 12, 12), ACT_RELU, 101),
    ("c116_ragged_f32", 116, 116, 116, (3, 13, 21), ACT_RELU, 2),
    ("c64_lrelu", 64, 64, 96, (1, 17, 9), ACT_LRELU, 101),
    ("c32_relu6_small", 48, 32, 40, (2, 5, 7), ACT_RELU6, 102),
    ("c128_none_f32", 96, 128, 112, (1, 20, 20), ACT_NONE, 2),
    # the benchmarked geometry: stage-2 and stage-3 units of ShuffleNetV2-1.0x at 320x320 input, more tiles than resident CTAs
    ("stage2_hw40", 58, 58, 58, (32, 40, 40), ACT_RELU, 101),
    ("stage3_hw20", 116, 116, 116, (48, 20, 20), ACT_RELU, 101),
]


@pytest.mark.parametrize("ucase", UNIT_CASES, ids=[c[0] for c in UNIT_CASES])
def test_unit_plain_input_bit_exact(ctx, ucase):
    from gpu_support import bits
    from tensor_b200 import F32_NCHW, S8_NHWC, UnitInt8, nhwc_channels
    name, cin, cm, cout, (n, h, w), act, term2 = ucase
    pw1, dw, pw2, want = _chain(cin, cm, cout, n, h, w, act, term2, seed=1000 + len(name), act_param0=0.1 if act == ACT_LRELU else 0.0)
    l1, ld, l2 = _layer(ctx, pw1), _layer(ctx, dw), _layer(ctx, pw2)
    unit = UnitInt8(ctx, l1, ld, l2)
    x = nchw_to_nhwc_padded(pw1.x_s8, nhwc_channels(cin))
    x[..., cin:] = 33  # whatever lies in the padding channels must not matter
    xd = ctx.to_device(x)
    out_dtype = S8_NHWC if term2 > 100 else F32_NCHW
    out = l2.out_array(n, h, w, out_dtype)
    od = ctx.malloc(out.nbytes)
    ctx.memset(od, 0x5A, out.nbytes)
    try:
        for _ in range(2):
            unit.forward_io(n, h, w, od, out_dtype, in_dev=xd)
        got = ctx.to_host(od, out.shape, out.dtype)
        if term2 > 100:
            assert not got[..., cout:].any()
            got = nhwc_padded_to_nchw(got, cout)
        assert np.array_equal(bits(got), bits(want))
    finally:
        ctx.free(xd)
        ctx.free(od)
        unit.close()
        for l in (l1, ld, l2):
            l.close()


def test_unit_gathered_input_and_mixed_output(ctx):
    """The form the graph uses: the first layer's channels gathered from three int8 tensors in shuffled order, the last layer
    storing per-channel-scaled int8 plus fp32 planes for some channels."""
    from gpu_support import bits
    from tensor_b200 import S8_NHWC, UnitInt8, nhwc_channels
    rng = np.random.default_rng(5)
    n, h, w, c = 5, 40, 40, 58
    src_ch = [58, 58, 116]
    picks = [(0, 29, 29), (1, 0, 15), (2, 70, 14)]
    chan_src = np.concatenate([np.full(cnt, s) for s, _, cnt in picks]).astype(np.int32)
    chan_idx = np.concatenate([np.arange(f, f + cnt) for _, f, cnt in picks]).astype(np.int32)
    perm = rng.permutation(chan_src.size)
    chan_src, chan_idx = chan_src[perm], chan_idx[perm]
    sources = [rng.integers(-127, 128, size=(n, cc, h, w), dtype=np.int8) for cc in src_ch]
    pw1, dw, pw2, _ = _chain(c, c, c, n, h, w, ACT_RELU, 101, seed=77)
    pw1.x_s8 = np.ascontiguousarray(np.stack([sources[s][:, ch] for s, ch in zip(chan_src, chan_idx)], axis=1))
    y1 = run_port(pw1, 0, want_acc=False)["y"]
    dw.x_s8 = y1
    _rescale(dw)
    y2 = run_port(dw, 0, want_acc=False)["y"]
    pw2.x_s8 = y2
    _rescale(pw2)
    f32_channels = sorted(rng.choice(c, size=c // 3, replace=False).tolist())
    scales = np.full(c, pw2.out_scales[0], np.float32) * rng.uniform(0.5, 1.5, c).astype(np.float32)
    scales[f32_channels] = 0.0
    pw2.out_scales = scales
    want_s8 = run_port(pw2, 0, want_acc=False)["y"]
    fcase = copy.copy(pw2)
    fcase.int8_scale_term, fcase.out_scales = 1, np.zeros(1, np.float32)
    want_f32 = run_port(fcase, 0, want_acc=False)["y"]

    l1 = _layer(ctx, pw1, gathered=(src_ch, chan_src, chan_idx))
    ld, l2 = _layer(ctx, dw), _layer(ctx, pw2)
    unit = UnitInt8(ctx, l1, ld, l2)
    ptrs = []
    for s, cc in zip(sources, src_ch):
        padded = nchw_to_nhwc_padded(s, nhwc_channels(cc))
        padded[..., cc:] = -9
        ptrs.append(ctx.to_device(padded))
    out = l2.out_array(n, h, w, S8_NHWC)
    od = ctx.malloc(out.nbytes)
    side = np.full((n, c, h, w), -12345.0, np.float32)
    sd = ctx.to_device(side)
    try:
        unit.forward_io(n, h, w, od, S8_NHWC, sources=ptrs, out_f32_dev=sd, f32_channels=f32_channels)
        got_s8 = nhwc_padded_to_nchw(ctx.to_host(od, out.shape, out.dtype), c)
        got_f32 = ctx.to_host(sd, side.shape, side.dtype)
        assert np.array_equal(got_s8, want_s8)
        assert np.array_equal(bits(got_f32[:, f32_channels]), bits(want_f32[:, f32_channels]))
        others = [ch for ch in range(c) if ch not in set(f32_channels)]
        assert (got_f32[:, others] == -12345.0).all()
    finally:
        for p in ptrs + [od, sd]:
            ctx.free(p)
        unit.close()
        for l in (l1, ld, l2):
            l.close()


def test_unit_refuses_what_it_cannot_fuse(ctx):
    from tensor_b200 import OtterB200Error, UnitInt8
    pw1, dw, pw2, _ = _chain(64, 64, 64, 1, 8, 8, ACT_RELU, 101, seed=3)
    wide1, wided, wide2, _ = _chain(64, 160, 64, 1, 8, 8, ACT_RELU, 101, seed=4)
    l1, ld, l2 = _layer(ctx, pw1), _layer(ctx, dw), _layer(ctx, pw2)
    w1, wd, w2 = _layer(ctx, wide1), _layer(ctx, wided), _layer(ctx, wide2)
    with pytest.raises(OtterB200Error):  # layers in the wrong order
        UnitInt8(ctx, ld, l1, l2)
    with pytest.raises(OtterB200Error):  # more channels between the layers than tensor memory holds
        UnitInt8(ctx, w1, wd, w2)
    for l in (l1, ld, l2, w1, wd, w2):
        l.close()
