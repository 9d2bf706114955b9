"""GPU: graphs built through the Net / Layer API mirror against the layer-by-layer CPU checker, bit-exact."""
import numpy as np
import pytest

from graph_walk import calibrate, walk
from tensor_b200 import graphs

pytestmark = pytest.mark.gpu


def bits(a):
    return a.view(np.int32) if a.dtype == np.float32 else a


def test_single_convolution_layer_net():
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    L = [dict(type="Input", name="data", output="data", channel=64, height=14, width=14),
         dict(type="Convolution", name="c1", input="data", output="c1", out_channels=128, kernel=1, int8_scale_term=102, activation="Relu"),
         dict(type="Convolution", name="c2", input="c1", output="c2", out_channels=128, kernel=3, padding=1, groups=128, int8_scale_term=101),
         dict(type="Convolution", name="c3", input="c2", output="c3", out_channels=64, kernel=1, int8_scale_term=2, activation="LRelu",
              activation_params="0.100000")]
    for l in L[1:]:  # the test helpers read the long option names
        k = l.pop("kernel")
        p = l.pop("padding", 0)
        l.update(kernel_h=k, kernel_w=k, stride_h=1, stride_w=1, padding_h=p, padding_w=p)
    params = graphs.make_params(L)
    x = np.random.default_rng(11).uniform(-1, 1, size=(3, 64, 14, 14)).astype(np.float32)
    calibrate(L, params, x, oracle_conv_for_calibration)
    want = walk(L, x, oracle_conv(params), want=["c1", "c2", "c3"])
    net = build_net(L, params)
    got = net.forward("data", x, ["c1", "c2", "c3"], dtypes=[np.int8, np.int8, np.float32])
    for name, g in zip(["c1", "c2", "c3"], got):
        assert np.array_equal(bits(g), bits(want[name])), name
    net.close()


def test_shufflenetv2_small_input_bit_exact():
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(64, 64, batch=2)
    params = graphs.make_params(L)
    x = np.random.default_rng(12).uniform(0, 1, size=(2, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration)
    probes = ["pool1", "s2b0_shuf", "s2b3_shuf", "s3b0_shuf", "s4b3_shuf", "conv5"]
    want = walk(L, x, oracle_conv(params), want=probes)
    net = build_net(L, params)
    got = net.forward("data", x, probes)
    for name, g in zip(probes, got):
        assert g.shape == want[name].shape, name
        assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
    # the default (lightmode) single-output path gives the same final blob
    again = net.forward("data", x, ["conv5"])[0]
    assert np.array_equal(bits(again), bits(want["conv5"]))
    net.close()


def test_int8_handover_between_convolutions_changes_no_blob():
    """pw1 -> dw -> pw2 chains hand their result over in int8 (no fp32 blob in between); every blob, the handed-over ones
    included, must still come out as the reference's fp32 values, and equal to a Net with the hand-over switched off."""
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(64, 64, batch=3)
    for l in L:  # a graph in which every convolution dequantizes: all blobs are fp32 in the reference
        if l["type"] == "Convolution" and int(l["int8_scale_term"]) > 100:
            l["int8_scale_term"] = int(l["int8_scale_term"]) - 100
    params = graphs.make_params(L, seed=77)
    x = np.random.default_rng(13).uniform(0, 1, size=(3, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration)
    probes = ["s2b0_l_dw", "s2b0_r_pw1", "s2b0_r_dw", "s2b1_pw1", "s2b1_dw", "s2b1_pw2", "s3b0_shuf", "s4b0_l_dw", "conv5"]
    want = walk(L, x, oracle_conv(params), want=probes)
    on = build_net(L, params)
    off = build_net(L, params, options={"int8_handover": 0})
    for net in (on, off):
        final = net.forward("data", x, ["conv5"])[0]
        assert np.array_equal(bits(final), bits(want["conv5"]))
        got = net.forward("data", x, probes)
        for name, g in zip(probes, got):
            assert g.dtype == np.float32 and g.shape == want[name].shape, name
            assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
    # never more kernels than with the switch off (where a layer cannot quantize its own input, a quantize pass goes away)
    counts = []
    for net in (on, off):
        before = net.context().launch_count()
        net.forward("data", x, ["conv5"])
        counts.append(net.context().launch_count() - before)
    assert counts[0] <= counts[1], counts
    with pytest.raises(Exception):
        on.set_option("no_such_option", 1)
    on.close()
    off.close()


def test_int8_routing_through_glue_layers_changes_no_blob():
    """Inside a ShuffleNetV2 stage every unit's result reaches the next units through Concat / ChannelShuffle / Crop. With
    "int8_routing" the producers store those channels quantized for their one reader and the readers run without a
    quantize pass; the graph's outputs and every intermediate blob asked for must not change by a bit."""
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(64, 64, batch=3)
    params = graphs.make_params(L, seed=5)
    x = np.random.default_rng(21).uniform(0, 1, size=(3, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration)
    probes = ["s2b0_shuf", "s2b1_pw2", "s2b2_shuf", "s3b5_pw2", "s3b7_shuf", "s4b0_r_pw2", "s4b3_shuf", "conv5"]
    want = walk(L, x, oracle_conv(params), want=probes)
    on = build_net(L, params)
    off = build_net(L, params, options={"int8_routing": 0})
    counts = []
    for net in (on, off):
        before = net.context().launch_count()
        final = net.forward("data", x, ["conv5"])[0]
        counts.append(net.context().launch_count() - before)
        assert np.array_equal(bits(final), bits(want["conv5"]))
    # the 13 stride-1 units, the first units of the three stages (whose two branches read the same channels with the same
    # scale, one of them through a depthwise layer; the first of them reads the first layer's pooled output) and conv5 lose
    # their quantize pass
    assert counts[1] - counts[0] == 17, counts
    for net in (on, off):
        # blobs that hold routed channels come out in fp32 all the same (the Net computes them without routing)
        got = net.forward("data", x, probes)
        for name, g in zip(probes, got):
            assert g.dtype == np.float32 and g.shape == want[name].shape, name
            assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
        # and the routed path still works afterwards
        assert np.array_equal(bits(net.forward("data", x, ["conv5"])[0]), bits(want["conv5"]))
    # a larger input (several pixel tiles per layer): routed and plain agree
    L2 = graphs.shufflenetv2_layers(160, 160, batch=2)
    p2 = graphs.make_params(L2, seed=6)
    x2 = np.random.default_rng(22).uniform(0, 1, size=(2, 3, 160, 160)).astype(np.float32)
    a = build_net(L2, p2)
    b = build_net(L2, p2, options={"int8_routing": 0})
    ya, yb = a.forward("data", x2, ["conv5"])[0], b.forward("data", x2, ["conv5"])[0]
    assert np.array_equal(bits(ya), bits(yb)) and np.abs(ya).max() > 0
    for net in (on, off, a, b):
        net.close()


def test_unknown_layer_type_is_an_error_not_an_exit():
    from tensor_b200 import Net, OtterB200Error
    net = Net(0)
    net.add_layer(type="Input", name="d", output="d", channel=3, height=8, width=8)
    net.add_layer(type="NoSuchLayer", name="x", input="d")
    with pytest.raises(OtterB200Error) as e:
        net.compile()
    assert "Unknown layer type" in str(e.value)
    net.close()


@pytest.mark.parametrize("h,w,cout,act,stride", [(45, 71, 24, "LRelu", 2), (64, 64, 16, "Relu", 2), (33, 130, 22, "LRelu", 2),
                                                 (37, 50, 24, "LRelu", 1), (16, 16, 8, "Relu6", 1), (320, 320, 24, "Relu", 2)])
def test_first_layer_and_maxpool_fused_kernel(h, w, cout, act, stride):
    """conv1 -> pool1 runs as one kernel; the pooled blob must equal the layer-by-layer checker, including the reference's
    packed zero-padding rule (cout % 4 == 0) after an activation that leaves negative values."""
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    from tensor_b200 import OtterB200Error
    L = [dict(type="Input", name="data", output="data", channel=3, height=h, width=w),
         graphs._conv("conv1", "data", cout, 3, stride, 1, 2, act),
         dict(type="MaxPool", name="pool1", input="conv1", output="pool1", kernel_h=3, kernel_w=3, stride_h=2, stride_w=2, padding_h=1, padding_w=1)]
    params = graphs.make_params(L)
    x = (np.random.default_rng(21).uniform(0, 1, size=(2, 3, h, w)).astype(np.float32))
    calibrate(L, params, x[:1], oracle_conv_for_calibration)
    params["conv1"]["bias"] -= np.float32(0.3)  # push many outputs negative so the padding rule decides border maxima
    want = walk(L, x, oracle_conv(params))["pool1"]
    net = build_net(L, params)
    got = net.forward("data", x, ["pool1"])[0]
    assert got.shape == want.shape
    assert np.array_equal(bits(got), bits(want))
    with pytest.raises(OtterB200Error):  # conv1 only exists inside the fused kernel
        net.forward("data", x, ["conv1"])
    net.close()


def test_whole_graph_equals_the_reference_s_own_net(tmp_path):
    """A whole graph, read from a .otter file, against blobs frozen from the reference's own Net (not only against the
    layer-by-layer checker)."""
    from graph_support import wide_shufflenet_case
    from support import GOLDEN_DIR
    from tensor_b200 import Net
    gold = np.load(GOLDEN_DIR / "net_shufflenet_wide_small.npz")
    L, params, x, blobs = wide_shufflenet_case()
    path = tmp_path / "graph.otter"
    path.write_text(graphs.to_otter_text(L))
    net = Net(0)
    net.load_otter(path)
    for name, p in params.items():
        net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    got = net.forward("data", x, blobs)
    for b, g in zip(blobs, got):
        assert np.array_equal(bits(g), bits(gold[b])), b
    net.close()


@pytest.mark.parametrize("c,h,w,n,opts,sh,sw", [(8, 7, 9, 2, dict(stride="2.000000"), 2.0, 2.0), (5, 7, 9, 2, dict(stride="2.000000"), 2.0, 2.0),
                                                (4, 5, 3, 1, dict(stride="3.000000"), 3.0, 3.0), (8, 6, 10, 3, dict(stride="1.500000"), 1.5, 1.5),
                                                (6, 6, 10, 2, dict(stride="1.500000"), 1.5, 1.5),
                                                (12, 7, 11, 2, dict(stride="0", scale_height="2.500000", scale_width="1.300000"), 2.5, 1.3),
                                                (7, 7, 11, 1, dict(stride="0", scale_height="2.500000", scale_width="1.300000"), 2.5, 1.3),
                                                (16, 9, 13, 2, dict(stride="1.700000"), 1.7, 1.7), (2, 9, 13, 2, dict(stride="1.700000"), 1.7, 1.7),
                                                (96, 40, 40, 2, dict(stride="2.000000"), 2.0, 2.0)])
def test_nearest_upsample_layer_both_index_rules(c, h, w, n, opts, sh, sw):
    """Nearest Upsample through the Net: the source pixel follows the reference's packed rule for channel counts that are
    multiples of 4 and its plain rule otherwise (they part for fractional scale factors)."""
    from graph_support import oracle_upsample
    from tensor_b200 import Net
    x = np.random.default_rng(c * 1000 + h * 10 + w).normal(size=(n, c, h, w)).astype(np.float32)
    net = Net(0)
    net.add_layer(type="Input", name="data", output="data", channel=c, height=h, width=w)
    net.add_layer(type="Upsample", name="up", input="data", output="up", upsample_mode="nearest", **opts)
    net.compile()
    oh, ow = int(h * np.float32(sh)), int(w * np.float32(sw))
    assert net.blob_shape("up")[1:] == (c, oh, ow)
    got = net.forward("data", x, ["up"])[0]
    want = oracle_upsample(x, oh, ow, (float(np.float32(sh)), float(np.float32(sw))), 1 if c % 4 == 0 else 0, mode="nearest")
    assert np.array_equal(bits(got), bits(want))
    net.close()


@pytest.mark.parametrize("c,h,w,n", [(8, 7, 9, 2), (16, 2, 2, 1), (12, 20, 20, 3), (5, 7, 9, 2), (6, 2, 3, 1), (58, 10, 10, 2), (3, 1, 4, 1), (96, 40, 40, 2)])
def test_upsample_layer_both_rounding_rules(c, h, w, n):
    """Bilinear x2 Upsample through the Net: channel counts the reference would pack (multiples of 4) and ones it would not
    follow different coefficient and rounding rules; both must match the checker bit for bit."""
    from graph_support import oracle_upsample
    from tensor_b200 import Net
    x = np.random.default_rng(c * 1000 + h * 10 + w).normal(size=(n, c, h, w)).astype(np.float32)
    net = Net(0)
    net.add_layer(type="Input", name="data", output="data", channel=c, height=h, width=w)
    net.add_layer(type="Upsample", name="up", input="data", output="up", upsample_mode="bilinear", align_corner="false", stride="2.000000")
    net.compile()
    assert net.blob_shape("up")[1:] == (c, 2 * h, 2 * w)
    got = net.forward("data", x, ["up"])[0]
    want = oracle_upsample(x, 2 * h, 2 * w, 2.0, 1 if c % 4 == 0 else 0)
    assert np.array_equal(bits(got), bits(want))
    net.close()


def test_detector_graph_bit_exact():
    """NanoDet-Plus-style detector on the ShuffleNetV2-1.0x widths (58/116/232-wide layers, 96-wide Ghost-PAN neck, depthwise
    5x5, Upsample, ShortCut, four heads), batch 2, against the layer-by-layer checker."""
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration, oracle_upsample
    L = graphs.nanodet_plus_layers(96, 128, batch=2)
    params = graphs.make_params(L, seed=31)
    x = np.random.default_rng(32).uniform(0, 1, size=(2, 3, 96, 128)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration, upsample_fn=oracle_upsample)
    probes = ["r8", "up32", "td16", "td8", "dn8", "bu32", "p64"] + list(graphs.NANODET_OUTPUTS)
    want = walk(L, x, oracle_conv(params), want=probes, upsample_fn=oracle_upsample)
    net = build_net(L, params)
    got = net.forward("data", x, probes)
    for name, g in zip(probes, got):
        assert g.shape == want[name].shape, name
        assert np.array_equal(bits(g), bits(want[name])), f"blob {name} differs"
    heads = net.forward("data", x, list(graphs.NANODET_OUTPUTS))
    for name, g in zip(graphs.NANODET_OUTPUTS, heads):
        assert np.array_equal(bits(g), bits(want[name])), name
    net.close()


def test_detector_graph_equals_the_reference_s_own_net(tmp_path):
    """The detector graph, read from a .otter file, against blobs frozen from the reference's own Net."""
    from graph_support import wide_nanodet_case
    from support import GOLDEN_DIR
    from tensor_b200 import Net
    gold = np.load(GOLDEN_DIR / "net_nanodet_wide_small.npz")
    L, params, x, blobs = wide_nanodet_case()
    path = tmp_path / "detector.otter"
    path.write_text(graphs.to_otter_text(L))
    net = Net(0)
    net.load_otter(path)
    for name, p in params.items():
        net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    got = net.forward("data", x, blobs)
    for b, g in zip(blobs, got):
        assert np.array_equal(bits(g), bits(gold[b])), b
    net.close()


def test_model_from_otter_and_ncnn_weight_file(tmp_path):
    """Net::load_otter(Inference) + Net::load_weight(Ncnn): graph and parameters both come from files, as for a real model.
    The file layout is pinned on the CPU side by the reference's own reader."""
    from graph_support import wide_nanodet_case, write_ncnn_bin
    from support import GOLDEN_DIR
    from tensor_b200 import Net, OtterB200Error
    gold = np.load(GOLDEN_DIR / "net_nanodet_wide_small.npz")
    L, params, x, blobs = wide_nanodet_case()
    (tmp_path / "m.otter").write_text(graphs.to_otter_text(L))
    write_ncnn_bin(L, params, tmp_path / "m.bin")
    net = Net(0)
    net.load_model(tmp_path / "m.otter", tmp_path / "m.bin", "ncnn")
    got = net.forward("data", x, blobs)
    for b, g in zip(blobs, got):
        assert np.array_equal(bits(g), bits(gold[b])), b
    net.close()
    # a file with bytes left over, or too short, is refused (the reference returns non-zero for both)
    data = (tmp_path / "m.bin").read_bytes()
    (tmp_path / "long.bin").write_bytes(data + b"\0\0\0\0")
    (tmp_path / "short.bin").write_bytes(data[:-8])
    for bad in ("long.bin", "short.bin"):
        net = Net(0)
        with pytest.raises(OtterB200Error):
            net.load_model(tmp_path / "m.otter", tmp_path / bad, "ncnn")
        net.close()


def test_detection_decode_kernel_batch():
    """ott_nanodet_detect on a batch of random head blobs against the C checker, image by image (tolerance: see
    graph_support.assert_same_detections)."""
    import ctypes as C
    from graph_support import assert_same_detections, oracle_detect
    from tensor_b200 import Context
    rng = np.random.default_rng(77)
    n, grids, strides = 3, (40, 20, 10, 5), [8, 16, 32, 64]
    heads = [(rng.normal(size=(n, 112, g, g)) * 2.0 - 2.5).astype(np.float32) for g in grids]
    with Context(0) as ctx:
        dev = []
        for hd in heads:
            p = ctx.malloc(hd.nbytes)
            ctx.check(ctx.lib.ott_memcpy_h2d(ctx.h, C.c_void_p(p), hd.ctypes.data, hd.nbytes))
            dev.append(p)
        ptrs = (C.c_void_p * 4)(*dev)
        gh = np.array(grids, np.int32)
        st = np.array(strides, np.int32)
        max_det = 2125
        out = np.zeros((n, max_det, 6), np.float32)
        counts = np.zeros(n, np.int32)
        ctx.check(ctx.lib.ott_nanodet_detect(ctx.h, ptrs, gh.ctypes.data, gh.ctypes.data, st.ctypes.data, 4, n, 80, 8, 0.4, 0.5,
                                             out.ctypes.data, counts.ctypes.data, max_det))
        for img in range(n):
            want = oracle_detect(heads, strides, image=img)
            assert counts[img] == want.shape[0] and counts[img] > 10
            assert_same_detections(out[img, :counts[img]], want)
        # max_det smaller than the number of detections: the count is still reported, the rows are truncated
        small = np.zeros((n, 5, 6), np.float32)
        ctx.check(ctx.lib.ott_nanodet_detect(ctx.h, ptrs, gh.ctypes.data, gh.ctypes.data, st.ctypes.data, 4, n, 80, 8, 0.4, 0.5,
                                             small.ctypes.data, counts.ctypes.data, 5))
        assert np.array_equal(small[0], out[0, :5]) and counts[0] > 5
        for p in dev:
            ctx.free(p)


def test_detection_decode_many_proposals_per_image():
    """One image whose proposals (6400: every cell of an 80x80 level passes the threshold) exceed what the per-image sort /
    NMS kernel holds in shared memory, next to one with a handful: the first is finished on the host, the second on the GPU,
    both equal the checker."""
    import ctypes as C
    from graph_support import assert_same_detections, oracle_detect
    from tensor_b200 import Context
    rng = np.random.default_rng(78)
    n, grids, strides = 2, (80,), [8]
    head = (rng.normal(size=(n, 112, 80, 80)) * 2.0).astype(np.float32)
    head[0, :80] += 3.0   # image 0: every cell's best class logit is well above the threshold
    head[1, :80] -= 7.0   # image 1: hardly any
    with Context(0) as ctx:
        p = ctx.malloc(head.nbytes)
        ctx.check(ctx.lib.ott_memcpy_h2d(ctx.h, C.c_void_p(p), head.ctypes.data, head.nbytes))
        ptrs = (C.c_void_p * 1)(p)
        gh = np.array(grids, np.int32)
        st = np.array(strides, np.int32)
        max_det = 6400
        out = np.zeros((n, max_det, 6), np.float32)
        counts = np.zeros(n, np.int32)
        ctx.check(ctx.lib.ott_nanodet_detect(ctx.h, ptrs, gh.ctypes.data, gh.ctypes.data, st.ctypes.data, 1, n, 80, 8, 0.4, 0.5,
                                             out.ctypes.data, counts.ctypes.data, max_det))
        for img in range(n):
            want = oracle_detect([head], strides, image=img)
            assert counts[img] == want.shape[0], (img, counts[img], want.shape)
            assert_same_detections(out[img, :counts[img]], want)
        assert counts[0] > 10 and counts[1] > 0, counts
        ctx.free(p)


def test_detector_with_decode_layer_from_files(tmp_path):
    """The whole detector including the NanodetPlusDetectionOutput layer, graph and weights from files; the detections against
    the reference's own decode of the reference's own head blobs (frozen)."""
    from graph_support import assert_same_detections, wide_nanodet_case, write_ncnn_bin
    from support import GOLDEN_DIR
    from tensor_b200 import Net
    gold = np.load(GOLDEN_DIR / "net_nanodet_wide_small.npz")
    L, params, x, _ = wide_nanodet_case()
    L = L + graphs.nanodet_plus_layers(64, 64, detect=True)[-1:]
    (tmp_path / "m.otter").write_text(graphs.to_otter_text(L))
    write_ncnn_bin(L, params, tmp_path / "m.bin")
    net = Net(0)
    net.load_model(tmp_path / "m.otter", tmp_path / "m.bin", "ncnn")
    rows, count = net.forward_rows("data", x, "nanodet")
    assert count == gold["detections"].shape[0] and count >= 1
    assert_same_detections(rows, gold["detections"])
    net.close()


def test_captured_forward_replays_bit_exact():
    """ott_net_capture: one forward frozen into a CUDA graph. Replays must give the bytes of the ordinary forward for whatever
    the input buffer holds at launch time, also after other forwards have gone through the same allocator in between."""
    import ctypes as C
    from graph_support import build_net, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(64, 64, batch=4)
    params = graphs.make_params(L, seed=5)
    rng = np.random.default_rng(6)
    x1 = rng.uniform(0, 1, size=(4, 3, 64, 64)).astype(np.float32)
    x2 = rng.uniform(0, 1, size=(4, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x1[:1], oracle_conv_for_calibration)
    net = build_net(L, params)
    ctx = net.context()
    blobs = ["conv5", "s2b1_shuf", "s3b0_l_dw"]  # a dense fp32 blob, a plane table (materialised), an int8 blob
    dtypes = [np.float32, np.float32, np.int8]
    want1 = net.forward("data", x1, blobs, dtypes=dtypes)
    want2 = net.forward("data", x2, blobs, dtypes=dtypes)
    din = ctx.malloc(x1.nbytes)
    graph = net.capture("data", C.c_void_p(din), x1.shape, blobs)

    def replay(x):
        ctx.check(ctx.lib.ott_memcpy_h2d(ctx.h, C.c_void_p(din), x.ctypes.data, x.nbytes))
        before = ctx.launch_count()
        graph.launch()
        assert ctx.launch_count() - before > 50  # the kernels inside the graph are counted
        outs = []
        for i, dt in enumerate(dtypes):
            ptr, shape = graph.output(i)
            if dt == np.int8:  # int8 blobs are NHWC with the channel stride padded to 16
                n, c, h, w = shape
                raw = np.empty((n, h, w, (c + 15) // 16 * 16), np.int8)
                ctx.check(ctx.lib.ott_memcpy_d2h(ctx.h, raw.ctypes.data, C.c_void_p(ptr), raw.nbytes))
                ctx.sync()
                outs.append(np.ascontiguousarray(raw[..., :c].transpose(0, 3, 1, 2)))
            else:
                a = np.empty(shape, np.float32)
                ctx.check(ctx.lib.ott_memcpy_d2h(ctx.h, a.ctypes.data, C.c_void_p(ptr), a.nbytes))
                ctx.sync()
                outs.append(a)
        return outs

    for x, want in ((x1, want1), (x2, want2)):
        for g, w_ in zip(replay(x), want):
            assert np.array_equal(bits(g), bits(w_))
    # other work through the same allocator must not get the graph's buffers
    net.forward("data", np.concatenate([x2, x1]), ["conv5"])
    for g, w_ in zip(replay(x1), want1):
        assert np.array_equal(bits(g), bits(w_))
    graph.close()
    ctx.free(din)
    net.close()


def test_chunked_host_forward_equals_plain_forward():
    """Large host batches run in chunks (captured forwards, overlapped copies); every image must come out as in a plain
    forward, on the first call (which captures), on later calls (which replay, with other data), after a parameter change
    (which must drop the captured forwards) and for an int8 output (which takes the plain path)."""
    from graph_support import build_net, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(32, 32, stage_repeats=(2, 2, 2))
    params = graphs.make_params(L)
    rng = np.random.default_rng(31)
    x = rng.uniform(0, 1, size=(150, 3, 32, 32)).astype(np.float32)
    calibrate(L, params, x[:1], oracle_conv_for_calibration)
    net = build_net(L, params)
    net2 = build_net(L, params, options={"host_chunk": 32})

    def plain(a):  # 50 < 2 * 64: no chunking
        return np.concatenate([net.forward("data", a[i:i + 50], ["conv5"])[0] for i in range(0, a.shape[0], 50)])

    whole = net.forward("data", x, ["conv5"])[0]              # chunks of 64, 64, 22
    assert np.array_equal(bits(whole), bits(plain(x)))
    assert np.array_equal(bits(net2.forward("data", x, ["conv5"])[0]), bits(whole))  # chunks of 32, ..., 22
    y = rng.uniform(0, 1, size=x.shape).astype(np.float32)
    assert np.array_equal(bits(net.forward("data", y, ["conv5"])[0]), bits(plain(y)))  # replay with other data
    two = net.forward("data", x, ["s2b1_shuf", "conv5"])      # two outputs, one of them a plane table
    assert np.array_equal(bits(two[1]), bits(whole))
    s8 = net.forward("data", x, ["s2b1_dw"], dtypes=[np.int8])[0]  # int8 NHWC blob: plain path, twice
    assert np.array_equal(s8, net.forward("data", x, ["s2b1_dw"], dtypes=[np.int8])[0])
    assert np.array_equal(s8[:50], net.forward("data", x[:50], ["s2b1_dw"], dtypes=[np.int8])[0])
    p = params["conv5"]
    net.set_conv_params("conv5", p["weight"], p["bias"] + np.float32(1.0), p["w_scales"], p["in_scales"], p["out_scales"])
    changed = net.forward("data", x, ["conv5"])[0]
    assert not np.array_equal(changed, whole) and np.array_equal(bits(changed), bits(plain(x)))
    net.close()
    net2.close()
