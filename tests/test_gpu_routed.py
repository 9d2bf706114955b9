"""GPU parity of the two building blocks of the int8 hand-over through Concat / Crop / ChannelShuffle, through the C-ABI:
a layer that reads its input channels from several int8 tensors (ott_conv_int8_create_gathered) and a requantizing launch
that also stores chosen channels as fp32 planes (ott_conv_int8_forward_io). Bit-exact against the CPU checker."""
import numpy as np
import pytest

from support import ACT_NONE, ACT_RELU, ACT_RELU6, ConvCase, nchw_to_nhwc_padded, nhwc_padded_to_nchw, run_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


def _layer(ctx, case, **kw):
    from tensor_b200 import ConvInt8
    return ConvInt8(ctx, cin=case.cin, cout=case.cout, kh=1, kw=1, bias_term=case.bias_term, int8_scale_term=case.int8_scale_term,
                    act_type=case.act_type, act_param0=case.act_param0, rounding=0, weight=case.weight,
                    bias=case.bias if case.bias_term else None, w_scales=case.w_scales, in_scales=case.in_scales,
                    out_scales=case.out_scales if case.requant else None, **kw)


# (source channel counts, [(source, first channel, count) in the order of the layer's input channels], cout, term, act)
GATHER_CASES = [
    ("two_halves", [58, 58], [(0, 29, 29), (1, 29, 29)], 58, 101, ACT_RELU),
    ("three_ranges_f32", [58, 116, 40], [(1, 30, 31), (0, 29, 29), (2, 5, 10)], 96, 1, ACT_NONE),
    ("tail_block_past_end", [232, 240], [(0, 200, 32), (1, 100, 140)], 232, 101, ACT_RELU6),
    ("single_source_whole", [64], [(0, 0, 64)], 128, 101, ACT_RELU),
    ("eight_sources", [116] * 8, [(s, 7 * s, 9 + s) for s in range(8)], 116, 2, ACT_RELU),
    # the benchmarked geometry: a stage-2 unit (58 channels, 40x40) and a stage-3 unit (116 channels, 20x20) of ShuffleNetV2-1.0x at
    # 320x320 input, with batches that give 800 / 600 pixel tiles, more than twice the CTAs resident on 148 SMs: every
    # persistent CTA walks over several tiles and the two-CTA-per-SM plans are taken
    ("stage2_unit_hw40", [58, 58, 58], [(0, 29, 29), (1, 0, 15), (2, 43, 14)], 58, 102, ACT_RELU, (64, 40, 40)),
    ("stage3_unit_hw20", [116] * 4, [(0, 87, 29), (1, 58, 29), (2, 29, 29), (3, 0, 29)], 116, 2, ACT_RELU, (192, 20, 20)),
]


@pytest.mark.parametrize("gcase", GATHER_CASES, ids=[c[0] for c in GATHER_CASES])
def test_gathered_input_bit_exact(ctx, gcase):
    from gpu_support import bits
    from tensor_b200 import F32_NCHW, KERNEL_DENSE_UMMA, S8_NHWC, nhwc_channels
    name, src_ch, picks, cout, term, act = gcase[:6]
    rng = np.random.default_rng(len(name) * 1000 + cout)
    n, h, w = gcase[6] if len(gcase) > 6 else (3, 13, 21)
    sources = [rng.integers(-127, 128, size=(n, c, h, w), dtype=np.int8) for c in src_ch]
    chan_src = np.concatenate([np.full(cnt, s) for s, _, cnt in picks]).astype(np.int32)
    chan_idx = np.concatenate([np.arange(f, f + cnt) for _, f, cnt in picks]).astype(np.int32)
    # interleave the logical channel order, as a ChannelShuffle does
    perm = rng.permutation(chan_src.size)
    chan_src, chan_idx = chan_src[perm], chan_idx[perm]
    case = ConvCase(name, int(chan_src.size), cout, 1, n=n, h=h, w=w, int8_scale_term=term, act_type=act, s8_input=True, seed=77).make()
    case.x_s8 = np.ascontiguousarray(np.stack([sources[s][:, c] for s, c in zip(chan_src, chan_idx)], axis=1))
    want = run_port(case, 0, want_acc=False)["y"]

    layer = _layer(ctx, case, gathered=(src_ch, chan_src, chan_idx))
    assert layer.kernel_kind == KERNEL_DENSE_UMMA
    ptrs = []
    try:
        for s, c in zip(sources, src_ch):
            padded = nchw_to_nhwc_padded(s, nhwc_channels(c))
            padded[..., c:] = 55  # what lies in the padding channels must not matter
            ptrs.append(ctx.to_device(padded))
        out_dtype = S8_NHWC if case.requant else F32_NCHW
        out = layer.out_array(n, h, w, out_dtype)
        out_dev = ctx.malloc(out.nbytes)
        layer.forward_io(n, h, w, out_dev, out_dtype, sources=ptrs)
        got = ctx.to_host(out_dev, out.shape, out.dtype)
        ctx.free(out_dev)
        if case.requant:
            got = nhwc_padded_to_nchw(got, cout)
        assert np.array_equal(bits(got), bits(want))
        # an ordinary forward of a gathered layer is refused
        from tensor_b200 import OtterB200Error
        with pytest.raises(OtterB200Error):
            layer.forward(ptrs[0], S8_NHWC, n, h, w, ptrs[0], out_dtype)
    finally:
        for p in ptrs:
            ctx.free(p)
        layer.close()


def test_gathered_rejects_bad_layouts(ctx):
    from tensor_b200 import OtterB200Error
    case = ConvCase("bad", 8, 32, 1, n=1, h=4, w=4, int8_scale_term=1, s8_input=True).make()
    with pytest.raises(OtterB200Error):  # the same source channel twice
        _layer(ctx, case, gathered=([64], np.zeros(8, np.int32), np.array([1, 1, 2, 3, 4, 5, 6, 7], np.int32)))
    with pytest.raises(OtterB200Error):  # a source narrower than one K block
        _layer(ctx, case, gathered=([8], np.zeros(8, np.int32), np.arange(8, dtype=np.int32)))
    with pytest.raises(OtterB200Error):  # channel index past the source
        _layer(ctx, case, gathered=([64], np.zeros(8, np.int32), np.arange(60, 68, dtype=np.int32)))


@pytest.mark.parametrize("cin,cout,act,s8_in", [(64, 58, ACT_RELU, True), (116, 116, ACT_NONE, False), (256, 512, ACT_RELU6, True)])
def test_fp32_side_output(ctx, cin, cout, act, s8_in):
    """int8 output with per-channel scales (0 for the fp32 channels) plus fp32 planes for a subset of the channels: the int8
    tensor equals that of the plain int8 launch, the chosen planes equal the fp32-output layer's, the others stay untouched."""
    from gpu_support import bits
    from tensor_b200 import F32_NCHW, S8_NHWC, nhwc_channels
    rng = np.random.default_rng(cin + cout)
    n, h, w = 2, 11, 17
    case = ConvCase("mixed", cin, cout, 1, n=n, h=h, w=w, int8_scale_term=101, act_type=act, s8_input=s8_in, seed=5).make()
    f32_channels = sorted(rng.choice(cout, size=cout // 3, replace=False).tolist())
    scales = np.full(cout, case.out_scales[0], np.float32) * rng.uniform(0.5, 1.5, cout).astype(np.float32)
    scales[f32_channels] = 0.0
    case.out_scales = scales
    want_s8 = run_port(case, 0, want_acc=False)["y"]
    import copy
    fcase = copy.copy(case)
    fcase.int8_scale_term = 1
    fcase.out_scales = np.zeros(1, np.float32)
    want_f32 = run_port(fcase, 0, want_acc=False)["y"]

    layer = _layer(ctx, case)
    x = nchw_to_nhwc_padded(case.x_s8, nhwc_channels(cin)) if s8_in else case.x_f32
    x_dev = ctx.to_device(x)
    out = layer.out_array(n, h, w, S8_NHWC)
    out_dev = ctx.malloc(out.nbytes)
    side = np.full((n, cout, h, w), -12345.0, np.float32)
    side_dev = ctx.to_device(side)
    try:
        layer.forward_io(n, h, w, out_dev, S8_NHWC, in_dev=x_dev, in_dtype=S8_NHWC if s8_in else F32_NCHW, out_f32_dev=side_dev,
                         f32_channels=f32_channels)
        got_s8 = nhwc_padded_to_nchw(ctx.to_host(out_dev, out.shape, out.dtype), cout)
        got_f32 = ctx.to_host(side_dev, side.shape, side.dtype)
        assert np.array_equal(got_s8, want_s8)
        assert not got_s8[:, f32_channels].any()
        assert np.array_equal(bits(got_f32[:, f32_channels]), bits(want_f32[:, f32_channels]))
        others = [c for c in range(cout) if c not in set(f32_channels)]
        assert (got_f32[:, others] == -12345.0).all()
    finally:
        for p in (x_dev, out_dev, side_dev):
            ctx.free(p)
        layer.close()


DW_GATHER_CASES = [
    ("s2_three_sources", [58, 58, 116], [(0, 0, 8), (1, 0, 7), (2, 0, 58)], 3, 2),
    ("s1_ranges_mid_group", [116, 232], [(1, 100, 60), (0, 20, 30)], 3, 1),
    ("k5_s2", [64, 64], [(0, 3, 20), (1, 40, 24)], 5, 2),
    # the benchmarked geometry: the stride-2 depthwise layers that open stages 3 and 4 of ShuffleNetV2-1.0x at 320x320 input
    # (116 channels at 40x40, 232 at 20x20), their channels spread over the previous stage's producers
    ("stage3_first_dw_hw40", [58, 58, 58], [(0, 0, 29), (1, 0, 29), (2, 0, 58)], 3, 2, (16, 40, 40)),
    ("stage4_first_dw_hw20", [116, 116, 116], [(0, 0, 58), (1, 0, 58), (2, 0, 116)], 3, 2, (24, 20, 20)),
    ("stage2_unit_dw_hw40", [58], [(0, 0, 58)], 3, 1, (16, 40, 40)),
]


@pytest.mark.parametrize("dcase", DW_GATHER_CASES, ids=[c[0] for c in DW_GATHER_CASES])
def test_gathered_depthwise_bit_exact(ctx, dcase):
    """A depthwise layer whose channels come from several int8 tensors: it runs over whole 16-channel groups of its sources
    and writes its output in that order; the logical channels, read back through the reported positions, equal the checker."""
    from tensor_b200 import ConvInt8, S8_NHWC, nhwc_channels
    name, src_ch, picks, k, stride = dcase[:5]
    rng = np.random.default_rng(len(name) + k)
    n, h, w = dcase[5] if len(dcase) > 5 else (2, 23, 37)
    sources = [rng.integers(-127, 128, size=(n, c, h, w), dtype=np.int8) for c in src_ch]
    chan_src = np.concatenate([np.full(cnt, s) for s, _, cnt in picks]).astype(np.int32)
    chan_idx = np.concatenate([np.arange(f, f + cnt) for _, f, cnt in picks]).astype(np.int32)
    perm = rng.permutation(chan_src.size)
    chan_src, chan_idx = chan_src[perm], chan_idx[perm]
    C_ = int(chan_src.size)
    case = ConvCase(name, C_, C_, k, stride=stride, pad=k // 2, groups=C_, n=n, h=h, w=w, int8_scale_term=101, act_type=ACT_RELU,
                    w_std=0.1, s8_input=True, seed=31).make()
    case.x_s8 = np.ascontiguousarray(np.stack([sources[s][:, c] for s, c in zip(chan_src, chan_idx)], axis=1))
    want = run_port(case, 0, want_acc=False)["y"]
    layer = ConvInt8(ctx, cin=C_, cout=C_, kh=k, kw=k, sh=stride, sw=stride, ph=k // 2, pw=k // 2, groups=C_, bias_term=1,
                     int8_scale_term=101, act_type=ACT_RELU, rounding=0, weight=case.weight, bias=case.bias, w_scales=case.w_scales,
                     in_scales=case.in_scales, out_scales=case.out_scales, gathered=(src_ch, chan_src, chan_idx))
    stored, pos = layer.gathered_layout()
    assert stored % 16 == 0 and stored >= C_ and len(set(pos.tolist())) == C_ and pos.max() < stored
    ptrs = []
    try:
        for s, c in zip(sources, src_ch):
            padded = nchw_to_nhwc_padded(s, nhwc_channels(c))
            padded[..., c:] = -77
            ptrs.append(ctx.to_device(padded))
        oh, ow = layer.out_hw(h, w)
        out_dev = ctx.malloc(n * oh * ow * stored)
        layer.forward_io(n, h, w, out_dev, S8_NHWC, sources=ptrs)
        got = ctx.to_host(out_dev, (n, oh, ow, stored), np.int8)
        ctx.free(out_dev)
        assert np.array_equal(np.ascontiguousarray(got[..., pos].transpose(0, 3, 1, 2)), want)
        rest = np.setdiff1d(np.arange(stored), pos)
        assert not got[..., rest].any()
    finally:
        for p in ptrs:
            ctx.free(p)
        layer.close()


@pytest.mark.parametrize("h,w,cout,stride,pad_zero", [(45, 71, 24, 2, 1), (64, 64, 16, 2, 0), (33, 40, 22, 1, 1)])
def test_first_layer_maxpool_int8_output(ctx, h, w, cout, stride, pad_zero):
    """The fused first layer + max-pool kernel with quantized output: float2int8(pooled * scale[c]) of exactly the fp32 values
    its fp32 form stores (that form is checked against the CPU checker elsewhere)."""
    import ctypes as C
    from tensor_b200 import ConvInt8, nhwc_channels
    n = 2
    case = ConvCase("stem", 3, cout, 3, stride=stride, pad=1, n=n, h=h, w=w, int8_scale_term=2, act_type=ACT_RELU, x_lo=0.0, seed=3).make()
    rng = np.random.default_rng(h + cout)
    scales = rng.uniform(5.0, 60.0, cout).astype(np.float32)
    kw = dict(cin=3, cout=cout, kh=3, kw=3, sh=stride, sw=stride, ph=1, pw=1, bias_term=1, act_type=ACT_RELU, rounding=0, weight=case.weight,
              bias=case.bias, w_scales=case.w_scales, in_scales=case.in_scales)
    f32_layer = ConvInt8(ctx, int8_scale_term=2, **kw)
    s8_layer = ConvInt8(ctx, int8_scale_term=101, out_scales=scales, **kw)
    oh, ow = f32_layer.out_hw(h, w)
    ph, pw = (oh - 1) // 2 + 1, (ow - 1) // 2 + 1
    cp = nhwc_channels(cout)
    x_dev = ctx.to_device(case.x_f32)
    f_dev, q_dev = ctx.malloc(n * cout * ph * pw * 4), ctx.malloc(n * ph * pw * cp)
    try:
        ctx.check(ctx.lib.ott_conv_int8_forward_maxpool(ctx.h, f32_layer.h, C.c_void_p(x_dev), n, h, w, pad_zero, C.c_void_p(f_dev)))
        ctx.check(ctx.lib.ott_conv_int8_forward_maxpool_s8(ctx.h, s8_layer.h, C.c_void_p(x_dev), n, h, w, pad_zero, C.c_void_p(q_dev)))
        pooled = ctx.to_host(f_dev, (n, cout, ph, pw), np.float32)
        got = ctx.to_host(q_dev, (n, ph, pw, cp), np.int8)
        t = pooled * scales[None, :, None, None]  # fp32 products, as __fmul_rn
        want = np.clip(np.trunc(t + np.copysign(np.float32(0.5), t)), -127, 127).astype(np.int8)
        assert np.array_equal(nhwc_padded_to_nchw(got, cout), want) and np.abs(want).max() > 5
        assert not got[..., cout:].any()
    finally:
        for p in (x_dev, f_dev, q_dev):
            ctx.free(p)
        f32_layer.close()
        s8_layer.close()


@pytest.mark.parametrize("cin,cout", [(64, 96), (128, 250)])
def test_scattered_int8_output(ctx, cin, cout):
    """Every 16-channel chunk of the int8 output goes to its own destination (tensor, channel offset, pitch); fp32 planes of
    chosen channels go where the plane map says. Same bytes as the plain launch."""
    from gpu_support import bits
    from tensor_b200 import S8_NHWC, nhwc_channels
    rng = np.random.default_rng(cin * cout)
    n, h, w = 2, 9, 31
    case = ConvCase("scatter", cin, cout, 1, n=n, h=h, w=w, int8_scale_term=101, act_type=ACT_RELU, s8_input=True, seed=8).make()
    case.out_scales = np.full(cout, case.out_scales[0], np.float32) * rng.uniform(0.5, 1.5, cout).astype(np.float32)
    want = run_port(case, 0, want_acc=False)["y"]
    import copy
    fcase = copy.copy(case)
    fcase.int8_scale_term, fcase.out_scales = 1, np.zeros(1, np.float32)
    want_f32 = run_port(fcase, 0, want_acc=False)["y"]
    layer = _layer(ctx, case)
    cp = nhwc_channels(cout)
    nch, pixels = cp // 16, n * h * w
    # three destination tensors of different widths; chunks dealt round-robin, one chunk dropped, two neighbours kept adjacent
    widths = [48, 32 * ((nch + 2) // 3), 16 * nch]
    bufs = [ctx.malloc(pixels * wd) for wd in widths]
    for b, wd in zip(bufs, widths):
        ctx.memset(b, 0x11, pixels * wd)
    used = [0, 0, 0]
    dst, pitch, where = [], [], []
    for c in range(nch):
        t = 0 if c < 2 else (1 if c % 2 else 2)
        if c == nch - 1 or used[t] + 16 > widths[t]:
            dst.append(0); pitch.append(0); where.append(None)
            continue
        dst.append(bufs[t] + used[t]); pitch.append(widths[t]); where.append((t, used[t]))
        used[t] += 16
    f32_channels = sorted(rng.choice(cout, size=cout // 4, replace=False).tolist())
    planes_total = cout + 7
    plane_of = rng.permutation(planes_total)[:cout]
    layer.set_f32_plane_map(plane_of, planes_total)
    side = np.full((n, planes_total, h, w), -7.0, np.float32)
    side_dev = ctx.to_device(side)
    x_dev = ctx.to_device(nchw_to_nhwc_padded(case.x_s8, nhwc_channels(cin)))
    try:
        layer.forward_io(n, h, w, 0, S8_NHWC, in_dev=x_dev, chunk_dst=dst, chunk_pitch=pitch, out_f32_dev=side_dev, f32_channels=f32_channels)
        got = [ctx.to_host(b, (pixels, wd), np.int8) for b, wd in zip(bufs, widths)]
        ref = nchw_to_nhwc_padded(want, cp).reshape(pixels, cp)
        for c, wh in enumerate(where):
            if wh is not None:
                assert np.array_equal(got[wh[0]][:, wh[1]:wh[1] + 16], ref[:, 16 * c:16 * c + 16]), c
        for t in range(3):
            assert (got[t][:, used[t]:] == 0x11).all()  # nothing written past the chunks placed there
        got_f32 = ctx.to_host(side_dev, side.shape, np.float32)
        for c in f32_channels:
            assert np.array_equal(bits(got_f32[:, plane_of[c]]), bits(want_f32[:, c])), c
        untouched = np.setdiff1d(np.arange(planes_total), plane_of[f32_channels])
        assert (got_f32[:, untouched] == -7.0).all()
    finally:
        for p in bufs + [side_dev, x_dev]:
            ctx.free(p)
        layer.close()
