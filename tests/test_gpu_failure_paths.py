"""GPU: the failure paths, exercised without faulting, trapping or hanging anything.

A kernel that gives up a bounded wait must surface as OTT_ERR_DEVICE_WAIT at the next synchronisation, once, and leave
the context usable; an allocation failure must surface as -100 (the reference's code for it, Tensor/Layer.cpp:50-59)
from the layer call and from the Net call, and the next call must succeed. The wait that runs out belongs to a probe
kernel that owns nothing (no copy in flight, no tensor memory); the allocation failure is injected on the host.
"""
import ctypes as C
import time

import numpy as np
import pytest

from support import ACT_RELU, ConvCase, rounding_for, run_port

pytestmark = pytest.mark.gpu

ERR_DEVICE_WAIT, ERR_ALLOC = -4, -100


@pytest.fixture()
def ctx():
    from tensor_b200 import Context
    with Context(0) as c:
        yield c


def _case():
    return ConvCase("failpath_pw", 64, 128, 1, n=2, h=12, w=12, int8_scale_term=101, act_type=ACT_RELU, seed=301).make()


def test_wait_that_runs_out_is_reported_once_and_the_context_survives(ctx):
    from gpu_support import bits, run_gpu
    lib = ctx.lib
    assert lib.ott_set_wait_limit_ms(ctx.h, 0) == -2  # a limit must be positive
    ctx.check(lib.ott_set_wait_limit_ms(ctx.h, 5))
    t0 = time.perf_counter()
    ctx.check(lib.ott_debug_wait_probe(ctx.h))
    rc = lib.ott_sync(ctx.h)
    waited = time.perf_counter() - t0
    assert rc == ERR_DEVICE_WAIT
    assert "0x100" in lib.ott_last_error(ctx.h).decode()
    assert waited < 1.5, f"a 5 ms wait limit took {waited:.2f} s to run out"
    # reported once: the word was cleared, the stream is alive
    assert lib.ott_sync(ctx.h) == 0
    # and the real kernels still run, with the short limit in force, and are still right
    case = _case()
    got, want = run_gpu(ctx, case, rounding_for("packed")), run_port(case, rounding_for("packed"))
    assert np.array_equal(got["acc"], want["acc"])
    assert np.array_equal(bits(got["y"]), bits(want["y"]))
    ctx.check(lib.ott_set_wait_limit_ms(ctx.h, 2000))


def test_host_entry_point_reports_a_pending_wait_failure(ctx):
    """The *_host forward synchronises itself: a status word left by an earlier kernel comes out of it."""
    from gpu_support import make_layer
    from tensor_b200 import F32_NCHW, S8_NHWC
    lib = ctx.lib
    case = _case()
    layer = make_layer(ctx, case, 0)
    want = layer.forward_host(case.x_f32, F32_NCHW, S8_NHWC)
    ctx.check(lib.ott_set_wait_limit_ms(ctx.h, 5))
    ctx.check(lib.ott_debug_wait_probe(ctx.h))
    out = np.empty_like(want)
    rc = lib.ott_conv_int8_forward_host(ctx.h, layer.h, case.x_f32.ctypes.data_as(C.c_void_p), F32_NCHW, case.n, case.h, case.w,
                                        out.ctypes.data_as(C.c_void_p), S8_NHWC)
    assert rc == ERR_DEVICE_WAIT
    again = layer.forward_host(case.x_f32, F32_NCHW, S8_NHWC)
    assert np.array_equal(again, want)
    layer.close()


def test_allocation_failure_in_a_layer_forward(ctx):
    from gpu_support import make_layer
    from tensor_b200 import F32_NCHW, S8_NHWC
    lib = ctx.lib
    case = _case()
    layer = make_layer(ctx, case, 0)
    want = layer.forward_host(case.x_f32, F32_NCHW, S8_NHWC)
    out = np.empty_like(want)
    for nth in (1, 2, 3):  # the input block, the output block, the scratch of the quantized activations
        ctx.check(lib.ott_debug_fail_alloc_after(ctx.h, nth))
        rc = lib.ott_conv_int8_forward_host(ctx.h, layer.h, case.x_f32.ctypes.data_as(C.c_void_p), F32_NCHW, case.n, case.h, case.w,
                                            out.ctypes.data_as(C.c_void_p), S8_NHWC)
        assert rc == ERR_ALLOC, (nth, rc)
        assert "alloc" in lib.ott_last_error(ctx.h).decode().lower()
    ctx.check(lib.ott_debug_fail_alloc_after(ctx.h, 0))
    stats = ctx.alloc_stats()
    assert stats["bytes_in_use"] >= 0
    assert np.array_equal(layer.forward_host(case.x_f32, F32_NCHW, S8_NHWC), want)
    # a failing create leaves nothing behind either
    before = ctx.alloc_stats()["bytes_in_use"]
    ctx.check(lib.ott_debug_fail_alloc_after(ctx.h, 2))
    with pytest.raises(Exception) as e:
        make_layer(ctx, case, 0)
    assert "-100" in str(e.value)
    ctx.check(lib.ott_debug_fail_alloc_after(ctx.h, 0))
    assert ctx.alloc_stats()["bytes_in_use"] == before
    layer.close()


def test_allocation_failure_in_a_net_forward():
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    from tensor_b200 import OtterB200Error, graphs
    from graph_walk import calibrate, walk
    L = graphs.shufflenetv2_layers(32, 32, batch=1, stage_repeats=(2, 2, 2))
    params = graphs.make_params(L, seed=9)
    x = np.random.default_rng(31).uniform(0, 1, size=(1, 3, 32, 32)).astype(np.float32)
    calibrate(L, params, x, oracle_conv_for_calibration)
    want = walk(L, x, oracle_conv(params))["conv5"]
    net = build_net(L, params)
    ctx = net.context()
    assert np.array_equal(net.forward("data", x, ["conv5"])[0].view(np.int32), want.view(np.int32))
    for nth in (1, 4, 9):
        ctx.check(ctx.lib.ott_debug_fail_alloc_after(ctx.h, nth))
        with pytest.raises(OtterB200Error) as e:
            net.forward("data", x, ["conv5"])
        assert e.value.code == ERR_ALLOC, (nth, e.value)
    ctx.check(ctx.lib.ott_debug_fail_alloc_after(ctx.h, 0))
    assert np.array_equal(net.forward("data", x, ["conv5"])[0].view(np.int32), want.view(np.int32))
    net.close()
