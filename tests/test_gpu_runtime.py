"""GPU tests of the runtime pieces: standalone quantize kernel, caching allocator, events, error paths."""
import ctypes as C

import numpy as np
import pytest

from support import ROUND_ADD_HALF_TRUNC, ROUND_HALF_AWAY, GOLDEN_DIR, _p, load_port, nhwc_padded_to_nchw

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


@pytest.mark.parametrize("n,c,h,w,per_channel", [(2, 64, 14, 14, False), (1, 3, 33, 31, False), (3, 58, 5, 7, True),
                                                  (1, 256, 56, 56, True), (2, 24, 1, 1, False), (1, 130, 9, 4, False),
                                                  (2, 704, 6, 6, True), (1, 1100, 3, 4, False)])
@pytest.mark.parametrize("rounding", [ROUND_ADD_HALF_TRUNC, ROUND_HALF_AWAY])
def test_quantize_matches_oracle(ctx, n, c, h, w, per_channel, rounding):
    from tensor_b200 import nhwc_channels
    rng = np.random.default_rng(7 + c)
    x = rng.uniform(-1, 1, size=(n, c, h, w)).astype(np.float32)
    scales = (rng.uniform(50, 200, size=c) if per_channel else np.array([127.0 / np.abs(x).max()])).astype(np.float32)
    want = np.empty(x.shape, np.int8)
    load_port().orc_quantize(_p(x, C.c_float), n, c, h, w, _p(scales, C.c_float), scales.size, rounding, _p(want, C.c_int8))
    xd = ctx.to_device(x)
    cp = nhwc_channels(c)
    od = ctx.malloc(n * h * w * cp)
    ctx.memset(od, 0x55, n * h * w * cp)
    ctx.quantize(xd, n, c, h, w, scales, rounding, od)
    got = ctx.to_host(od, (n, h, w, cp), np.int8)
    ctx.free(xd)
    ctx.free(od)
    assert np.array_equal(nhwc_padded_to_nchw(got, c), want)
    assert not got[..., c:].any()


def test_quantize_rounding_ties(ctx):
    adv = np.load(GOLDEN_DIR / "epilogue_adversarial.npz")
    ties = adv["ties"]  # [8,4,68] treated as one image c=8,h=4,w=68 by the reference
    ok = np.abs(ties) < 2.0e9
    for tag, rounding in (("packed", ROUND_ADD_HALF_TRUNC), ("unpacked", ROUND_HALF_AWAY)):
        xd = ctx.to_device(ties)
        od = ctx.malloc(4 * 68 * 16)
        ctx.quantize(xd, 1, 8, 4, 68, np.ones(1, np.float32), rounding, od)
        got = nhwc_padded_to_nchw(ctx.to_host(od, (1, 4, 68, 16), np.int8), 8)[0]
        ctx.free(xd)
        ctx.free(od)
        assert np.array_equal(got[ok], adv[f"ties_q_{tag}"][ok]), tag


def test_caching_allocator_reuses_blocks(ctx):
    s0 = ctx.alloc_stats()
    a = ctx.malloc(3 << 20)
    ctx.free(a)
    b = ctx.malloc(3 << 20)
    s1 = ctx.alloc_stats()
    assert b == a, "a freed block of the same rounded size must be handed out again"
    assert s1["cache_hits"] >= s0["cache_hits"] + 1
    ctx.free(b)
    # steady state: repeated same-shape forwards must not reach cudaMalloc again
    from cases import small_cases
    from gpu_support import run_gpu
    case = [c for c, _ in small_cases() if c.name == "pw_64_256_relu6_s8"][0].make()
    run_gpu(ctx, case, 0)
    m0 = ctx.alloc_stats()["device_mallocs"]
    for _ in range(3):
        run_gpu(ctx, case, 0)
    assert ctx.alloc_stats()["device_mallocs"] == m0


def test_events_time_the_stream(ctx):
    e0, e1 = ctx.event(), ctx.event()
    p = ctx.malloc(64 << 20)
    ctx.record(e0)
    ctx.memset(p, 1, 64 << 20)
    ctx.record(e1)
    assert ctx.elapsed_ms(e0, e1) > 0.0
    ctx.free(p)
    ctx.lib.ott_event_destroy(e0)
    ctx.lib.ott_event_destroy(e1)


def test_argument_errors_are_reported(ctx):
    from tensor_b200 import ConvInt8, OtterB200Error
    w = np.zeros((8, 8, 1, 1), np.int8)
    one = np.ones(8, np.float32)
    with pytest.raises(OtterB200Error):  # sigmoid epilogue is not bit-reproducible: refused, not approximated
        ConvInt8(ctx, cin=8, cout=8, kh=1, kw=1, act_type=4, weight=w, bias=one, w_scales=one, in_scales=one[:1])
    with pytest.raises(OtterB200Error):  # fp32 layer has no int8 path
        ConvInt8(ctx, cin=8, cout=8, kh=1, kw=1, int8_scale_term=0, weight=w, bias=one, w_scales=one, in_scales=one[:1])
    with pytest.raises(OtterB200Error):  # grouped but not depthwise
        ConvInt8(ctx, cin=8, cout=8, kh=1, kw=1, groups=2, weight=np.zeros((8, 4, 1, 1), np.int8), bias=one, w_scales=one, in_scales=one[:1])
    layer = ConvInt8(ctx, cin=8, cout=8, kh=1, kw=1, int8_scale_term=2, weight=w, bias=one, w_scales=one, in_scales=one[:1])
    from tensor_b200 import F32_NCHW, S8_NHWC
    with pytest.raises(OtterB200Error):  # int8 output from a layer without top_blob_int8_scales
        layer.forward_host(np.zeros((1, 8, 4, 4), np.float32), F32_NCHW, S8_NHWC)
    layer.close()


@pytest.mark.parametrize("name,kw", [
    ("pw", dict(cin=64, cout=64, k=1, int8_scale_term=101, act_type=1)),
    ("dense3x3", dict(cin=64, cout=64, k=3, pad=1, int8_scale_term=2)),
    ("dw_f32in", dict(cin=32, cout=32, k=3, pad=1, groups=32, int8_scale_term=101, w_std=0.1)),
    ("dw_s8in", dict(cin=58, cout=58, k=3, pad=1, groups=58, int8_scale_term=101, w_std=0.1, s8_input=True)),
    ("stem", dict(cin=3, cout=24, k=3, stride=2, pad=1, int8_scale_term=2, act_type=1, x_lo=0.0)),
])
def test_empty_batch_and_single_pixel(ctx, name, kw):
    """Edges of the batch and map sizes: a call with zero images succeeds and launches nothing (the output buffer is not
    touched); a 1 x 1 map (all padding around one pixel) equals the CPU checker."""
    from gpu_support import bits, make_layer, run_gpu
    from support import ConvCase, run_port
    from tensor_b200 import F32_NCHW, S8_NHWC
    case = ConvCase("edge_" + name, n=1, h=1, w=1, seed=77, **kw).make()
    want = run_port(case, 0, want_acc=False)["y"]
    got = run_gpu(ctx, case, 0, want_acc=False)["y"]
    assert np.array_equal(bits(got), bits(want))
    layer = make_layer(ctx, case, 0)
    try:
        in_dtype = S8_NHWC if case.s8_input else F32_NCHW
        out_dtype = S8_NHWC if case.requant else F32_NCHW
        buf = ctx.malloc(4096)
        ctx.memset(buf, 0x5A, 4096)
        before = ctx.launch_count()
        layer.forward(buf, in_dtype, 0, 7, 9, buf + 2048, out_dtype)
        ctx.sync()
        assert ctx.launch_count() == before
        assert (ctx.to_host(buf, (4096,), np.uint8) == 0x5A).all()
        ctx.free(buf)
    finally:
        layer.close()
