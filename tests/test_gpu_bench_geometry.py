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


@pytest.mark.parametrize("routing", [1, 0], ids=["routed", "unrouted"])
def test_shipped_detector_equals_the_reference_s_own_net(routing, tmp_path):
    """The detector the reference ships (benchmark/nanodet-plus-m-1.5x_416_int8_fused.otter: 1.5x widths, 416x416; the
    generated description equals that file layer for layer, tests/test_otter_format.py), read from a .otter file, seeded
    parameters: the four heads against what the reference's own Net computed for the same inputs (frozen fixture), bit for bit."""
    from graph_support import assert_equals_shipped_golden, shipped_nanodet_case
    from support import GOLDEN_DIR
    from tensor_b200 import Net
    gold = np.load(GOLDEN_DIR / "net_nanodet_shipped_416.npz")
    L, params, x, heads = shipped_nanodet_case()
    path = tmp_path / "shipped.otter"
    path.write_text(graphs.to_otter_text(L))
    net = Net(0)
    net.set_option("int8_routing", routing)
    net.load_otter(path)
    for name, p in params.items():
        net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    got = dict(zip(heads, net.forward("data", x, heads)))
    assert_equals_shipped_golden(got, gold)
    # the same through a batch of three copies: every image of a batch equals the single-image answer
    xb = np.ascontiguousarray(np.repeat(x, 3, axis=0))
    for name, g in zip(heads, net.forward("data", xb, heads)):
        for i in range(3):
            assert np.array_equal(bits(g[i]), bits(got[name][0])), f"head {name}, image {i}"
    net.close()


def test_shipped_mixed_detector_fp32_first_layer():
    """The "mixed" flavour of the shipped detector (..._int8_mixed.otter: conv_1 keeps fp32, int8_scale_term 0): the fp32 blob
    is within the fp32 layer's tolerance of float64 arithmetic, and all four heads equal the CPU checker fed with that blob."""
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration, oracle_upsample
    from test_f32_layer import TOL_ULP, activation, conv_f64
    L = graphs.shipped_nanodet_plus_layers(mixed=True, detect=False)
    conv1_name = next(l["name"] for l in L if l["type"] == "Convolution")
    rng = np.random.default_rng(4160)
    x = rng.uniform(0, 1, size=(1, 3, 416, 416)).astype(np.float32)
    w1 = rng.normal(0, 0.2, size=(24, 3, 3, 3)).astype(np.float32)
    b1 = rng.normal(0, 0.1, size=(24,)).astype(np.float32)
    exact, mag = conv_f64(x, w1, b1, 2, 1, 1, 1)
    conv1_f64 = activation(exact, 2, 0.1)
    params = graphs.make_params(L, seed=4161)
    int8_params = {k: v for k, v in params.items() if k != conv1_name}

    def first_layer_then(fn, conv1_blob):
        return lambda name, g, *a: conv1_blob(*a) if name == conv1_name else fn(name, g, *a)

    calibrate(L, params, x, first_layer_then(oracle_conv_for_calibration, lambda p, a, as_float: conv1_f64.astype(np.float32)),
              upsample_fn=oracle_upsample)
    net = build_net(L, int8_params)
    net.set_conv_params_f32(conv1_name, w1, b1)
    conv1 = net.forward("data", x, [conv1_name])[0]
    err = np.abs(conv1.astype(np.float64) - conv1_f64) / (mag * 2.0 ** -23 + 1e-30)
    assert err.max() <= TOL_ULP
    heads = list(graphs.NANODET_OUTPUTS)
    want = walk(L, x, first_layer_then(oracle_conv(params), lambda a: conv1), want=heads, upsample_fn=oracle_upsample)
    for name, g in zip(heads, net.forward("data", x, heads)):
        assert np.array_equal(bits(g), bits(want[name])), f"head {name} differs"
    net.close()


@pytest.mark.parametrize("routing", [1, 0], ids=["routed", "unrouted"])
def test_depthwise_pointwise_fusion_changes_no_blob(shufflenet_320, routing):
    """"fuse_depthwise_pointwise": every depthwise 3x3 layer whose only reader is a 1x1 layer runs inside that layer's kernel
    (plain and gathered inputs, stride 1 and 2, 24 to 232 channels, int8 + fp32 side outputs). Same bits at the benchmarked
    geometry, fewer launches; a depthwise layer's own blob can still be extracted (the pair then runs as two layers)."""
    from graph_support import build_net
    L, params, x, probes, want = shufflenet_320
    fused = build_net(L, params, options={"int8_routing": routing, "fuse_depthwise_pointwise": 1})
    plain = build_net(L, params, options={"int8_routing": routing})
    counts = []
    for net in (fused, plain):
        before = net.context().launch_count()
        got = net.forward("data", x, ["conv5"])[0]
        counts.append(net.context().launch_count() - before)
        assert np.array_equal(bits(got), bits(want["conv5"]))
    # routed: 18 of the 19 depthwise layers fuse (the one behind the first layer's 24-channel pooled output is laid out in
    # 16-channel groups, which the pair kernel does not read); unrouted: the 13 stride-1 units and the three right branches
    # (the left-branch depthwise layers of the stride-2 units read fp32 blobs there and run by themselves)
    assert counts[1] - counts[0] == (18 if routing else 16), counts
    got = fused.forward("data", x, probes)
    for name, g in zip(probes, got):
        assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
    # a fused-away blob is still there for the asking, and the fused path still works afterwards
    dw_blob = fused.forward("data", x, ["s2b1_dw"])[0]
    ref_blob = plain.forward("data", x, ["s2b1_dw"])[0]
    assert dw_blob.shape == ref_blob.shape and np.array_equal(bits(dw_blob), bits(ref_blob))
    assert np.array_equal(bits(fused.forward("data", x, ["conv5"])[0]), bits(want["conv5"]))
    fused.close()
    plain.close()
