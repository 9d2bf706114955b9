"""Graph-level checker: the benchmark graphs executed layer by layer with the CPU checkers (convolutions through the
C restatement of the reference, glue layers in numpy as validated against the compiled reference)."""
from __future__ import annotations

import numpy as np

from support import ConvCase, run_port
from graph_walk import calibrate, walk
from tensor_b200 import graphs


def _case(name, g, p, a, term):
    c = ConvCase(name, g["cin"], g["cout"], g["k"], g["stride"], g["pad"], groups=g["groups"], n=a.shape[0], h=a.shape[2], w=a.shape[3],
                 bias_term=1, int8_scale_term=term, act_type=g["act"], act_param0=g["act_param0"], s8_input=(a.dtype == np.int8))
    c.weight, c.bias, c.w_scales = p["weight"], p["bias"], p["w_scales"]
    c.in_scales = p["in_scales"]
    c.out_scales = p["out_scales"] if term > 100 else np.zeros((1,), np.float32)
    if a.dtype == np.int8:
        c.x_s8, c.x_f32 = np.ascontiguousarray(a), None
    else:
        c.x_f32, c.x_s8 = np.ascontiguousarray(a, dtype=np.float32), None
    return c


def oracle_conv(params, rounding=0):
    def fn(name, g, a):
        return run_port(_case(name, g, params[name], a, g["term"]), rounding, want_acc=False)["y"]
    return fn


def oracle_upsample(a, oh, ow, scale, packed_rule, mode="bilinear"):
    """The C checker's Upsample (bilinear with exact fused multiply-adds, or nearest), for walk(upsample_fn=...)."""
    import ctypes as C
    from support import _p, load_port
    lib = load_port()
    fn = getattr(lib, "orc_upsample_" + mode)
    fn.restype = None
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double, C.c_double, C.c_int, C.c_void_p]
    a = np.ascontiguousarray(a, dtype=np.float32)
    n, c, h, w = a.shape
    y = np.empty((n, c, oh, ow), np.float32)
    sh, sw = scale if isinstance(scale, tuple) else (scale, scale)
    fn(a.ctypes.data, n, c, h, w, oh, ow, float(sh), float(sw), int(packed_rule), y.ctypes.data)
    return y


def oracle_detect(heads, strides, prob_threshold=0.4, nms_threshold=0.5, image=0, num_class=80):
    """The C checker's detection decode of one image: rows {label + 1, score, x, y, width, height}."""
    import ctypes as C
    from support import load_port
    lib = load_port()
    lib.orc_nanodet_detect.restype = C.c_int
    lib.orc_nanodet_detect.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p,
                                       C.c_int]
    one = [np.ascontiguousarray(h[image], dtype=np.float32) for h in heads]
    ptrs = (C.c_void_p * len(one))(*[h.ctypes.data for h in one])
    gh = np.array([h.shape[1] for h in one], np.int32)
    gw = np.array([h.shape[2] for h in one], np.int32)
    st = np.array(strides, np.int32)
    cells = int((gh * gw).sum())
    out = np.zeros((cells, 6), np.float32)
    n = lib.orc_nanodet_detect(ptrs, gh.ctypes.data, gw.ctypes.data, st.ctypes.data, len(one), num_class, (one[0].shape[0] - num_class) // 4,
                               prob_threshold, nms_threshold, out.ctypes.data, cells)
    return out[:n].copy()


def assert_same_detections(got, want, score_tol=3e-7, box_tol=3e-4):
    """Detection rows agree up to the documented floating-point tolerance of the decode (expf and divisions round differently
    in the reference's -Ofast build, the C checker and the GPU): same count, labels and order, scores and boxes close."""
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.array_equal(got[:, 0], want[:, 0])
    assert np.abs(got[:, 1] - want[:, 1]).max(initial=0) <= score_tol
    assert np.abs(got[:, 2:] - want[:, 2:]).max(initial=0) <= box_tol


def oracle_conv_for_calibration(name, g, p, a, as_float):
    term = g["term"] - 100 if (as_float and g["term"] > 100) else g["term"]
    return run_port(_case(name, g, p, a, term), 0, want_acc=False)["y"]


def build_net(layers, params, device=0, options=None):
    from tensor_b200 import Net
    net = Net(device)
    for key, value in (options or {}).items():
        net.set_option(key, value)
    for l in layers:
        net.add_layer(**l)
    net.compile()
    for name, p in params.items():
        net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    return net


def wide_shufflenet_case():
    """A ShuffleNetV2-shaped graph whose widths are all multiples of 8 (24 / 176 / 352 / 704, the 1.5x widths of the
    reference's own shipped graph), so that the reference's packed Net can run it whole; small input, one image."""
    L = graphs.shufflenetv2_layers(64, 64, stage_repeats=(2, 3, 2), stage_channels=(176, 352, 704), stem=24, last=512)
    params = graphs.make_params(L, seed=0x0771E5 + 15)
    x = np.random.default_rng(515).uniform(0, 1, size=(1, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x, oracle_conv_for_calibration)
    return L, params, x, ["pool1", "s2b1_shuf", "s3b2_shuf", "conv5"]


def wide_nanodet_case():
    """The detector graph (backbone + Ghost-PAN neck + four heads) with widths that are all multiples of 8, so that the
    reference's packed Net can run it whole; 64x64 input, one image: the levels are 8x8, 4x4, 2x2 and 1x1."""
    L = graphs.nanodet_plus_layers(64, 64, neck=96, stage_repeats=(2, 2, 2), stage_channels=(176, 352, 704))
    params = graphs.make_params(L, seed=0x0771E5 + 25)
    x = np.random.default_rng(525).uniform(0, 1, size=(1, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x, oracle_conv_for_calibration, upsample_fn=oracle_upsample)
    return L, params, x, ["up32", "td16", "td8", "bu16", "bu32", "p64"] + list(graphs.NANODET_OUTPUTS)


def shipped_nanodet_case():
    """The detector the reference ships (benchmark/nanodet-plus-m-1.5x_416_int8_fused.otter: 1.5x widths, 128 neck channels,
    416x416; graphs.shipped_nanodet_plus_layers is that file layer for layer) with seeded parameters, one image. Every width
    is a multiple of 8, so the reference's packed Net runs it whole."""
    L = graphs.shipped_nanodet_plus_layers(detect=False)
    params = graphs.make_params(L, seed=0x0771E5 + 416)
    x = np.random.default_rng(416).uniform(0, 1, size=(1, 3, 416, 416)).astype(np.float32)
    calibrate(L, params, x, oracle_conv_for_calibration, upsample_fn=oracle_upsample)
    return L, params, x, list(graphs.NANODET_OUTPUTS)


def write_ncnn_bin(layers, params, path):
    """The parameters as an ncnn model file, the way a quantized ncnn model stores them and ConvolutionLayer::load_model reads
    them back (Tensor/ConvolutionLayer.cpp:245-296): per Convolution, in graph order, the int8 weights behind the tag
    0x000D4B38 (padded to 4 bytes), the bias, the weight scales ([groups] for a depthwise layer with int8_scale_term 1/101,
    [out_channels] for a dense one), the scalar input scale and, for int8_scale_term > 100, the scalar output scale."""
    geo = graphs.conv_geometry(layers)
    with open(path, "wb") as f:
        for l in layers:
            if l["type"] != "Convolution":
                continue
            g, p = geo[l["name"]], params[l["name"]]
            w = np.ascontiguousarray(p["weight"], dtype=np.int8).tobytes()
            f.write(np.uint32(0x000D4B38).tobytes() + w + b"\0" * (-len(w) % 4))
            f.write(np.ascontiguousarray(p["bias"], dtype=np.float32).tobytes())
            f.write(np.ascontiguousarray(p["w_scales"], dtype=np.float32).tobytes())
            f.write(np.float32(p["in_scales"][0]).tobytes())
            if g["term"] > 100:
                f.write(np.float32(p["out_scales"][0]).tobytes())


def reference_net_forward(layers, params, x, blobs, packed=1, weight_file=None):
    """The same graph through the compiled reference's own Net (oracle/_ref): .otter text -> Net::load_otter -> parameters
    replaced -> Extractor. One image."""
    import ctypes as C
    import tempfile
    from support import _p, load_ref
    ref = load_ref()
    with tempfile.NamedTemporaryFile("w", suffix=".otter", delete=False) as f:
        f.write(graphs.to_otter_text(layers))
        path = f.name
    try:
        if weight_file is not None:  # parameters through the reference's own ncnn weight reader
            assert ref.ref_net_open_weights(path.encode(), str(weight_file).encode(), packed) == 0, ref.ref_last_error()
        else:
            assert ref.ref_net_open(path.encode(), packed) == 0, ref.ref_last_error()
        for name, p in ({} if weight_file is not None else params).items():
            os_ = p["out_scales"]
            rc = ref.ref_net_set_conv(name.encode(), _p(p["weight"], C.c_int8), _p(p["bias"], C.c_float), _p(p["w_scales"], C.c_float),
                                      _p(p["in_scales"], C.c_float), p["in_scales"].size, _p(os_, C.c_float) if os_ is not None else None,
                                      0 if os_ is None else os_.size)
            assert rc == 0, (name, ref.ref_last_error())
        out = {}
        for b in blobs:
            shape = np.zeros(4, np.int32)
            assert ref.ref_net_forward(b"data", _p(x, C.c_float), x.shape[1], x.shape[2], x.shape[3], b.encode(), None, _p(shape, C.c_int)) == 0
            y = np.empty(tuple(shape), np.float32)
            assert ref.ref_net_forward(b"data", _p(x, C.c_float), x.shape[1], x.shape[2], x.shape[3], b.encode(), _p(y, C.c_float), _p(shape, C.c_int)) == 0
            out[b] = y
        return out
    finally:
        ref.ref_net_close()
        import os
        os.unlink(path)


def assert_equals_shipped_golden(heads, gold):
    """heads: {name: fp32 array} of graph_support.shipped_nanodet_case; gold: tests/golden/net_nanodet_shipped_416.npz (the
    reference's own Net on that case). Bit for bit: full arrays where the fixture keeps them, SHA-256 of the bytes for all."""
    import hashlib
    for name in graphs.NANODET_OUTPUTS:
        a = np.ascontiguousarray(heads[name])
        assert tuple(a.shape) == tuple(gold[name + "_shape"]), name
        if name in gold.files:
            assert np.array_equal(a.view(np.int32), gold[name].view(np.int32)), f"head {name} differs from the reference's Net"
        assert hashlib.sha256(a.tobytes()).hexdigest() == gold[name + "_sha256"].tobytes().decode(), f"head {name}: digest differs"
