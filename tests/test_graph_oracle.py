"""CPU tests of the graph plumbing: the numpy glue layers against the compiled reference's own layers, shape
inference of the ShuffleNetV2 description, and the calibration walk."""
import ctypes as C

import numpy as np
import pytest

from support import _p, have_ref, load_ref
from graph_walk import calibrate, walk
from tensor_b200 import graphs


def ref_layer(type_, opts, ins, packed=1):
    ref = load_ref()
    n = len(ins)
    arr = (C.POINTER(C.c_float) * n)(*[_p(np.ascontiguousarray(a), C.c_float) for a in ins])
    shapes = np.array([d for a in ins for d in a.shape], np.int32)
    osh = np.zeros(4, np.int32)
    assert ref.ref_layer_forward(type_.encode(), opts.encode(), n, arr, _p(shapes, C.c_int), packed, None, _p(osh, C.c_int)) == 0
    out = np.empty(tuple(osh), np.float32)
    assert ref.ref_layer_forward(type_.encode(), opts.encode(), n, arr, _p(shapes, C.c_int), packed, _p(out, C.c_float), _p(osh, C.c_int)) == 0
    return out


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
def test_numpy_glue_equals_reference_layers():
    rng = np.random.default_rng(5)
    x = (rng.normal(size=(1, 24, 17, 19)) - 0.7).astype(np.float32)  # mostly negative: zero padding must win at the border
    layers = [dict(type="Input", name="d", output="d", channel=24, height=17, width=19),
              dict(type="MaxPool", name="p", input="d", output="p", kernel_h=3, kernel_w=3, stride_h=2, stride_w=2, padding_h=1, padding_w=1)]
    want = ref_layer("MaxPool", "kernel_h=3;kernel_w=3;stride_h=2;stride_w=2;padding_h=1;padding_w=1", [x])
    assert np.array_equal(walk(layers, x, None)["p"], want)
    x5 = np.ascontiguousarray(x[:, :5])  # 5 channels: not packed by the reference -> plain kernel, padding never wins
    want5 = ref_layer("MaxPool", "kernel_h=3;kernel_w=3;stride_h=2;stride_w=2;padding_h=1;padding_w=1", [x5])
    layers[0]["channel"] = 5
    assert np.array_equal(walk(layers, x5, None)["p"], want5)
    y = rng.normal(size=(1, 12, 4, 6)).astype(np.float32)
    z = rng.normal(size=(1, 12, 4, 6)).astype(np.float32)
    g = [dict(type="Input", name="a", output="a", channel=12, height=4, width=6),
         dict(type="ChannelShuffle", name="s", input="a", output="s", groups=2),
         dict(type="Crop", name="c", input="s", output="c", start=6, end=12, axis=1)]
    got = walk(g, y, None, want=["s", "c"])
    assert np.array_equal(got["s"], ref_layer("ChannelShuffle", "groups=2", [y]))
    assert np.array_equal(got["c"], ref_layer("Crop", "start=6;end=12;axis=1", [got["s"]]))
    assert np.array_equal(np.concatenate([y, z], 1), ref_layer("Concat", "axis=1", [y, z]))
    assert np.array_equal(y + z, ref_layer("ShortCut", "", [y, z]))
    assert np.array_equal(np.where(y < 0, y * np.float32(0.1), y), ref_layer("LRelu", "alpha=0.1", [y]))
    assert np.array_equal(np.clip(y * 4, 0, 6), ref_layer("Relu6", "", [y * 4]))


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
@pytest.mark.parametrize("c,h,w", [(8, 7, 9), (16, 2, 2), (4, 5, 3), (12, 20, 20), (5, 7, 9), (6, 2, 3), (58, 10, 10), (3, 1, 4), (96, 40, 40)])
def test_checker_upsample_equals_reference_layer(c, h, w):
    """The reference resizes packed blobs (C % 4 == 0) and plain blobs with different coefficient rules and rounding;
    the checker restates both. Sizes include the clamped borders (2 rows / columns) and one-row planes for the plain rule."""
    from graph_support import oracle_upsample
    x = np.random.default_rng(c * 1000 + h * 10 + w).normal(size=(1, c, h, w)).astype(np.float32)
    want = ref_layer("Upsample", "upsample_mode=bilinear;align_corner=false;stride=2.000000", [x])
    got = oracle_upsample(x, 2 * h, 2 * w, 2.0, 1 if c % 4 == 0 else 0)
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.int32), want.view(np.int32))
    if c % 4 == 0:  # the two rules really differ: the test above would not notice a swapped flag otherwise
        assert not np.array_equal(oracle_upsample(x, 2 * h, 2 * w, 2.0, 0), want) or h * w <= 4


NEAREST_CASES = [(8, 7, 9, "stride=2.000000", 2.0, 2.0), (5, 7, 9, "stride=2.000000", 2.0, 2.0), (4, 5, 3, "stride=3.000000", 3.0, 3.0),
                 (3, 5, 3, "stride=3.000000", 3.0, 3.0), (8, 6, 10, "stride=1.500000", 1.5, 1.5), (6, 6, 10, "stride=1.500000", 1.5, 1.5),
                 (12, 7, 11, "stride=0;scale_height=2.500000;scale_width=1.300000", 2.5, 1.3),
                 (7, 7, 11, "stride=0;scale_height=2.500000;scale_width=1.300000", 2.5, 1.3),
                 (16, 9, 13, "stride=1.700000", 1.7, 1.7), (2, 9, 13, "stride=1.700000", 1.7, 1.7), (4, 3, 5, "stride=1.000000", 1.0, 1.0)]


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
@pytest.mark.parametrize("c,h,w,opts,sh,sw", NEAREST_CASES)
def test_checker_nearest_upsample_equals_reference_layer(c, h, w, opts, sh, sw):
    """Nearest Upsample: the reference picks the source pixel by two different rules (packed / plain blob); fractional scale
    factors are where they part."""
    from graph_support import oracle_upsample
    x = np.random.default_rng(c * 1000 + h * 10 + w).normal(size=(1, c, h, w)).astype(np.float32)
    want = ref_layer("Upsample", "upsample_mode=nearest;" + opts, [x])
    oh, ow = int(h * np.float32(sh)), int(w * np.float32(sw))
    assert want.shape == (1, c, oh, ow)
    got = oracle_upsample(x, oh, ow, (float(np.float32(sh)), float(np.float32(sw))), 1 if c % 4 == 0 else 0, mode="nearest")
    assert np.array_equal(got.view(np.int32), want.view(np.int32))


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
def test_reference_upsample_ignores_align_corner_under_default_options():
    """With NetOption's defaults the reference's layer resizes through otter::Interpolate without handing align_corner on
    (Tensor/UpsampleLayer.cpp:120-121), so the flag changes nothing; the GPU layer relies on that."""
    x = np.random.default_rng(3).normal(size=(1, 8, 6, 5)).astype(np.float32)
    for c in (8, 5):
        a = ref_layer("Upsample", "upsample_mode=bilinear;align_corner=false;stride=2.000000", [x[:, :c]])
        b = ref_layer("Upsample", "upsample_mode=bilinear;align_corner=true;stride=2.000000", [x[:, :c]])
        assert np.array_equal(a.view(np.int32), b.view(np.int32))


def test_nanodet_plus_description():
    L = graphs.nanodet_plus_layers(320, 320)
    geo = graphs.conv_geometry(L)
    hw, macs = graphs.conv_input_hw(L, 320, 320)
    assert geo["r8"]["cin"] == 116 and geo["r32"]["cin"] == 464 and geo["td16_g1pw"]["cin"] == 192 and geo["td16_scdw"]["k"] == 5
    assert hw["head8"] == (40, 40) and hw["head16"] == (20, 20) and hw["head32"] == (10, 10) and hw["head64"] == (5, 5)
    assert all(geo[h]["cout"] == 80 + 4 * 8 for h in graphs.NANODET_OUTPUTS)
    assert sum(1 for l in L if l["type"] == "Upsample") == 2 and sum(1 for l in L if l["type"] == "ShortCut") == 5
    # every layer type of the graph is one the .otter writer/reader round-trips
    from tensor_b200 import capi
    back = capi.parse_otter_text(graphs.to_otter_text(L))
    assert [l["name"] for l in back] == [l["name"] for l in L]
    assert next(l for l in back if l["name"] == "up32")["upsample_mode"] == "bilinear"


def test_shufflenetv2_description():
    L = graphs.shufflenetv2_layers(320, 320)
    geo = graphs.conv_geometry(L)
    assert len(geo) == 2 + 3 * 5 + (3 + 7 + 3) * 3  # stem + conv5, 5 convs per down-sampling unit, 3 per basic unit
    assert geo["conv1"]["cin"] == 3 and geo["conv5"]["cin"] == 464 and geo["conv5"]["cout"] == 1024
    assert geo["s2b0_l_dw"]["groups"] == 24 and geo["s3b1_pw1"]["cin"] == 116 and geo["s4b3_dw"]["groups"] == 232
    # multiply-accumulates per image at 320x320 (ops = 2x): the figure the images/s bench converts to TOP/s
    macs, h = 0, {"data": 320}
    for l in L:
        ins = [s.strip() for s in str(l.get("input", "")).split(",") if s.strip()]
        if l["type"] == "Input":
            continue
        hin = h[ins[0]]
        if l["type"] in ("Convolution", "MaxPool"):
            k, s, p = int(l["kernel_h"]), int(l["stride_h"]), int(l["padding_h"])
            h[l["output"]] = (hin + 2 * p - k) // s + 1
            if l["type"] == "Convolution":
                g = geo[l["name"]]
                macs += h[l["output"]] ** 2 * g["cout"] * (g["cin"] // g["groups"]) * k * k
        else:
            h[l["output"]] = hin
    assert 2.5e8 < macs < 3.5e8, macs


def test_calibration_walk_gives_usable_scales():
    from graph_support import oracle_conv, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(32, 32, stage_repeats=(2, 2, 2))
    params = graphs.make_params(L)
    x = np.random.default_rng(3).uniform(0, 1, size=(1, 3, 32, 32)).astype(np.float32)
    calibrate(L, params, x, oracle_conv_for_calibration)
    out = walk(L, x, oracle_conv(params))["conv5"]
    assert out.shape == (1, 1024, 1, 1) and np.isfinite(out).all() and (out != 0).mean() > 0.2
    # an int8 blob's producer and consumer agree on its scale
    assert params["s2b1_pw1"]["out_scales"][0] == params["s2b1_dw"]["in_scales"][0]


NET_GOLD = np.load(__import__("support").GOLDEN_DIR / "net_shufflenet_wide_small.npz")


def test_layer_by_layer_walk_equals_frozen_reference_net():
    """The graph-level checker (C restatement per convolution + numpy glue) against blobs frozen from the reference's
    own Net on a whole graph."""
    from graph_support import oracle_conv, wide_shufflenet_case
    L, params, x, blobs = wide_shufflenet_case()
    got = walk(L, x, oracle_conv(params), want=blobs)
    for b in blobs:
        assert np.array_equal(got[b].view(np.int32), NET_GOLD[b].view(np.int32)), b


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
def test_reference_net_live_equals_walk():
    from graph_support import oracle_conv, reference_net_forward, wide_shufflenet_case
    L, params, x, blobs = wide_shufflenet_case()
    ref = reference_net_forward(L, params, x, blobs)
    got = walk(L, x, oracle_conv(params), want=blobs)
    for b in blobs:
        assert np.array_equal(got[b].view(np.int32), ref[b].view(np.int32)), b


DET_GOLD = np.load(__import__("support").GOLDEN_DIR / "net_nanodet_wide_small.npz")


def test_detector_walk_equals_frozen_reference_net():
    """Backbone + Ghost-PAN neck (bilinear Upsample, Concat, ShortCut, depthwise 5x5) + heads: the layer-by-layer checker
    against blobs frozen from the reference's own Net."""
    from graph_support import oracle_conv, oracle_upsample, wide_nanodet_case
    L, params, x, blobs = wide_nanodet_case()
    got = walk(L, x, oracle_conv(params), want=blobs, upsample_fn=oracle_upsample)
    for b in blobs:
        assert got[b].shape == DET_GOLD[b].shape, b
        assert np.array_equal(got[b].view(np.int32), DET_GOLD[b].view(np.int32)), b


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
def test_reference_detector_net_live_equals_frozen():
    from graph_support import reference_net_forward, wide_nanodet_case
    L, params, x, blobs = wide_nanodet_case()
    ref = reference_net_forward(L, params, x, blobs)
    for b in blobs:
        assert np.array_equal(ref[b].view(np.int32), DET_GOLD[b].view(np.int32)), b


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
def test_reference_reads_our_ncnn_weight_file(tmp_path):
    """The .bin written by the test helper, read by the reference's own Net::load_weight(…, Ncnn), gives the frozen blobs:
    pins the file layout that the GPU Net's reader is then tested against."""
    from graph_support import reference_net_forward, wide_nanodet_case, write_ncnn_bin
    L, params, x, blobs = wide_nanodet_case()
    path = tmp_path / "detector.bin"
    write_ncnn_bin(L, params, path)
    ref = reference_net_forward(L, params, x, blobs, weight_file=path)
    for b in blobs:
        assert np.array_equal(ref[b].view(np.int32), DET_GOLD[b].view(np.int32)), b


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
@pytest.mark.parametrize("seed,shift", [(3, -2.5), (4, -4.0), (5, -1.0)])
def test_checker_detection_decode_against_reference_layer(seed, shift):
    """NanodetPlusDetectionOutput: the restatement against the reference's own layer on random head blobs. Not bit-exact by
    nature (see assert_same_detections); counts, labels and order must agree."""
    from graph_support import assert_same_detections, oracle_detect
    rng = np.random.default_rng(seed)
    heads = [(rng.normal(size=(1, 112, g, g)) * 2.0 + shift).astype(np.float32) for g in (40, 20, 10, 5)]
    want = ref_layer("NanodetPlusDetectionOutput", "prob_threshold=0.4;nms_threshold=0.5;stride=8, 16, 32, 64", heads, packed=0).reshape(-1, 6)
    got = oracle_detect(heads, [8, 16, 32, 64])
    assert want.shape[0] > 10
    assert_same_detections(got, want)


def test_detections_of_the_frozen_reference_heads():
    """The decode of the head blobs frozen from the reference's own Net, against the reference's own decode of them."""
    from graph_support import assert_same_detections, oracle_detect
    heads = [DET_GOLD[k] for k in graphs.NANODET_OUTPUTS]
    got = oracle_detect(heads, [8, 16, 32, 64])
    assert got.shape[0] >= 1
    assert_same_detections(got, DET_GOLD["detections"])


def test_shipped_detector_walk_equals_frozen_reference_net():
    """The detector the reference ships (1.5x widths, 416x416, 190 layers), seeded parameters: the layer-by-layer checker
    against the heads frozen from the reference's own Net at that full geometry."""
    from graph_support import assert_equals_shipped_golden, oracle_conv, oracle_upsample, shipped_nanodet_case
    gold = np.load(__import__("support").GOLDEN_DIR / "net_nanodet_shipped_416.npz")
    L, params, x, heads = shipped_nanodet_case()
    got = walk(L, x, oracle_conv(params), want=heads, upsample_fn=oracle_upsample)
    assert_equals_shipped_golden(got, gold)


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")
def test_shipped_detector_reference_net_live_equals_fixture():
    from graph_support import assert_equals_shipped_golden, reference_net_forward, shipped_nanodet_case
    gold = np.load(__import__("support").GOLDEN_DIR / "net_nanodet_shipped_416.npz")
    L, params, x, heads = shipped_nanodet_case()
    assert_equals_shipped_golden(reference_net_forward(L, params, x, heads), gold)
