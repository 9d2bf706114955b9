"""The allocation-free forward against the ordinary one.

ott_conv_int8_forward_noalloc exists for hosts that cannot let the library reach cudaMalloc while they
run (device memory split into fixed pools at start-up, or a latency bound that cannot absorb the
device-wide synchronisation of an allocation). It must give exactly the bytes the ordinary forward gives.
Collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from support import ACT_RELU, ACT_RELU6, ConvCase

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 32 << 20  # OTT_NOALLOC_SCRATCH_BYTES in include/otter_b200.h


def _forward_both(ctx, case):
    """Returns (ordinary output, [no-alloc output of call 1, of call 2], device mallocs seen by the no-alloc calls)."""
    from gpu_support import make_layer
    from tensor_b200 import F32_NCHW, S8_NHWC
    layer = make_layer(ctx, case, 0)
    out_dtype = S8_NHWC if case.requant else F32_NCHW
    want = layer.forward_host(case.x_f32, F32_NCHW, out_dtype)
    xd = ctx.to_device(case.x_f32)
    od = ctx.malloc(want.nbytes)
    got = []
    mallocs_before = ctx.alloc_stats()["device_mallocs"]
    for fill in (0x11, 0xEE):  # two calls in a row; the output buffer is dirtied differently before each
        ctx.memset(od, fill, want.nbytes)
        rc = ctx.lib.ott_conv_int8_forward_noalloc(ctx.h, layer.h, C.c_void_p(xd), case.n, case.h, case.w, C.c_void_p(od), out_dtype)
        ctx.check(rc)
        ctx.sync()
        mallocs_after = ctx.alloc_stats()["device_mallocs"]
        got.append(ctx.to_host(od, want.shape, want.dtype))
    ctx.free(xd)
    ctx.free(od)
    layer.close()
    return want, got, mallocs_after - mallocs_before


@pytest.fixture(scope="module")
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


@pytest.mark.parametrize("case", [
    ConvCase("noalloc_pw_s8", 64, 256, 1, n=3, h=28, w=28, int8_scale_term=101, act_type=ACT_RELU6, seed=201),
    ConvCase("noalloc_3x3_f32", 64, 64, 3, 1, 1, n=2, h=20, w=24, int8_scale_term=2, seed=202),
    ConvCase("noalloc_dw_s8", 96, 96, 3, 2, 1, groups=96, n=2, h=21, w=19, int8_scale_term=101, act_type=ACT_RELU, w_std=0.1, seed=203),
    ConvCase("noalloc_stem_f32", 3, 24, 3, 2, 1, n=2, h=32, w=32, int8_scale_term=2, x_lo=0.0, seed=204),
], ids=lambda c: c.name)
def test_noalloc_forward_equals_ordinary_forward(ctx, case):
    case.make()
    want, got, new_mallocs = _forward_both(ctx, case)
    for i, g in enumerate(got):
        assert np.array_equal(g.view(np.uint8), want.view(np.uint8)), f"call {i + 1} differs from the ordinary forward"
    assert new_mallocs == 0, "the allocation-free entry point reached cudaMalloc through the context's allocator"


def test_noalloc_rejects_oversized_calls(ctx):
    from gpu_support import make_layer
    from tensor_b200 import S8_NHWC
    case = ConvCase("noalloc_big", 64, 64, 1, n=1, h=8, w=8, int8_scale_term=101, act_type=ACT_RELU, seed=205).make()
    layer = make_layer(ctx, case, 0)
    n = SCRATCH_BYTES // (8 * 8 * 64) + 1  # one image more than fits
    rc = ctx.lib.ott_conv_int8_forward_noalloc(ctx.h, layer.h, C.c_void_p(0x1000), n, 8, 8, C.c_void_p(0x1000), S8_NHWC)
    assert rc == -2
    msg = ctx.lib.ott_last_error(ctx.h).decode()
    assert str(SCRATCH_BYTES) in msg and "exceed" in msg
    layer.close()


def test_noalloc_refuses_before_it_launches_anything(ctx):
    """A call the convolution stage would refuse (a layer with gathered input, an output type the layer does not produce)
    must fail before the quantize kernel has been enqueued and the shared array overwritten."""
    from gpu_support import make_layer
    from tensor_b200 import ConvInt8, F32_NCHW, S8_NHWC
    case = ConvCase("noalloc_gathered", 58, 58, 1, n=1, h=8, w=8, int8_scale_term=101, act_type=ACT_RELU, s8_input=True, seed=206).make()
    gathered = ConvInt8(ctx, cin=58, cout=58, kh=1, kw=1, bias_term=1, int8_scale_term=101, act_type=ACT_RELU, weight=case.weight, bias=case.bias,
                        w_scales=case.w_scales, in_scales=case.in_scales, out_scales=case.out_scales,
                        gathered=([64], np.zeros(58, np.int32), np.arange(58, dtype=np.int32)))
    plain = make_layer(ctx, case, 0)
    x = ctx.malloc(58 * 8 * 8 * 4)
    o = ctx.malloc(64 * 8 * 8 * 4)
    before = ctx.launch_count()
    assert ctx.lib.ott_conv_int8_forward_noalloc(ctx.h, gathered.h, C.c_void_p(x), 1, 8, 8, C.c_void_p(o), S8_NHWC) == -2
    assert "gathered" in ctx.lib.ott_last_error(ctx.h).decode()
    assert ctx.lib.ott_conv_int8_forward_noalloc(ctx.h, plain.h, C.c_void_p(x), 1, 8, 8, C.c_void_p(o), F32_NCHW) == -2
    assert ctx.launch_count() == before
    ctx.free(x)
    ctx.free(o)
    gathered.close()
    plain.close()
