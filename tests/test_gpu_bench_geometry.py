"""GPU: the two graph workloads at the geometry the benchmark runs them on (320x320 input: feature maps of 80, 40, 20 and
10 pixels a side, pixel tiles in the thousands), against the layer-by-layer CPU checker, bit for bit, with the int8
hand-over through the glue layers on and off, through the ordinary forward, the captured (CUDA graph) forward the
benchmark replays, and the chunked host-buffer forward its end-to-end leg calls."""
import ctypes as C

import numpy as np
import pytest

from graph_walk import calibrate, walk
from tensor_b200 import graphs

pytestmark = pytest.mark.gpu


def bits(a):
    return a.view(np.int32) if a.dtype == np.float32 else a


@pytest.fixture(scope="module")
def shufflenet_320():
    from graph_support import oracle_conv, oracle_conv_for_calibration
    n = 4
    L = graphs.shufflenetv2_layers(320, 320, batch=n)
    params = graphs.make_params(L)
    x = np.random.default_rng(320).uniform(0, 1, size=(n, 3, 320, 320)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration)
    probes = ["pool1", "s2b3_shuf", "s3b7_shuf", "s4b3_shuf", "conv5"]  # one blob per stage and the output
    want = walk(L, x, oracle_conv(params), want=probes)
    return L, params, x, probes, want


@pytest.mark.parametrize("routing", [1, 0], ids=["routed", "unrouted"])
def test_shufflenetv2_at_320x320(shufflenet_320, routing):
    from graph_support import build_net
    L, params, x, probes, want = shufflenet_320
    net = build_net(L, params, options={"int8_routing": routing})
    final = net.forward("data", x, ["conv5"])[0]  # the benchmarked call: one output, routed where the option allows
    assert np.array_equal(bits(final), bits(want["conv5"]))
    got = net.forward("data", x, probes)
    for name, g in zip(probes, got):
        assert g.shape == want[name].shape, name
        assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
    net.close()


def test_shufflenetv2_at_320x320_captured_forward_and_host_pipeline(shufflenet_320):
    """What bench.py times: replays of the captured forward on a device batch, and ott_net_forward on pinned host buffers
    (64-image chunks, overlapped copies). A batch of 130 images made of the four checked ones, so that the chunked path
    runs three chunks with a ragged last one and every output row can be compared."""
    from graph_support import build_net
    L, params, x, probes, want = shufflenet_320
    n = 130
    xb = np.ascontiguousarray(x[np.arange(n) % x.shape[0]])
    net = build_net(graphs.shufflenetv2_layers(320, 320, batch=n), params)
    ctx = net.context()
    # captured forward on a device-resident batch
    din = ctx.to_device(xb)
    g = net.capture("data", C.c_void_p(din), xb.shape, ["conv5"])
    for _ in range(2):
        g.launch()
    ctx.sync()
    dptr, shp = g.output(0)
    got = ctx.to_host(dptr, tuple(shp), np.float32)
    for i in range(n):
        assert np.array_equal(bits(got[i]), bits(want["conv5"][i % x.shape[0]])), f"image {i} of the replayed forward differs"
    g.close()
    ctx.free(din)
    # host buffers in and out (pageable numpy memory works like pinned memory, only slower)
    out = net.forward("data", xb, ["conv5"])[0]
    for i in range(n):
        assert np.array_equal(bits(out[i]), bits(want["conv5"][i % x.shape[0]])), f"image {i} of the host-buffer forward differs"
    net.close()


@pytest.mark.parametrize("routing", [1, 0], ids=["routed", "unrouted"])
def test_detector_at_320x320(routing):
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration, oracle_upsample
    n = 2
    L = graphs.nanodet_plus_layers(320, 320, batch=n)
    params = graphs.make_params(L, seed=3200)
    x = np.random.default_rng(3201).uniform(0, 1, size=(n, 3, 320, 320)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration, upsample_fn=oracle_upsample)
    heads = list(graphs.NANODET_OUTPUTS)
    probes = ["s2b3_shuf", "s3b7_shuf", "s4b3_shuf", "td8", "bu32", "p64"] + heads
    want = walk(L, x, oracle_conv(params), want=probes, upsample_fn=oracle_upsample)
    net = build_net(L, params, options={"int8_routing": routing})
    got = net.forward("data", x, heads)  # the benchmarked call
    for name, g in zip(heads, got):
        assert np.array_equal(bits(g), bits(want[name])), f"head {name} differs"
    got = net.forward("data", x, probes)
    for name, g in zip(probes, got):
        assert g.shape == want[name].shape, name
        assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
    net.close()
