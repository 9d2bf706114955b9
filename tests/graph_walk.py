"""A graph interpreter on host numpy arrays, for the tests and for picking activation scales.

`walk` executes a layer list (tensor_b200.graphs) with a caller-supplied convolution function; the glue layers are done
here in numpy, validated against the compiled reference's own layers (test_graph_oracle.py). The parity tests pass the
CPU checker as the convolution; `calibrate` is also used by the benchmark's set-up, which passes the GPU library's own
layer to pick activation scales from one sample image. Test and set-up plumbing: not part of the shipped package.
"""
from __future__ import annotations

import numpy as np

from tensor_b200.graphs import conv_geometry


def maxpool_nchw(x, k, s, p, pad_zero):
    n, c, h, w = x.shape
    oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    fill = np.float32(0.0) if pad_zero else np.float32(-np.inf)
    xp = np.full((n, c, h + 2 * p, w + 2 * p), fill, np.float32)
    xp[:, :, p:p + h, p:p + w] = x
    out = np.full((n, c, oh, ow), -np.inf, np.float32)
    for ky in range(k):
        for kx in range(k):
            out = np.maximum(out, xp[:, :, ky:ky + s * oh:s, kx:kx + s * ow:s][:, :, :oh, :ow])
    return out


def upsample_bilinear_approx(a, oh, ow, scale, packed_rule):
    """Bilinear resize in float64, rounded once: good for picking calibration ranges, NOT bit-exact with the reference (the
    checker's exact version is the C function orc_upsample_bilinear; tests pass it to `walk` as upsample_fn)."""
    def taps(n_in, n_out):
        d = np.arange(n_out, dtype=np.float64)
        f = np.clip((d + 0.5) * (n_in / n_out) - 0.5, 0, n_in - 1)
        i0 = np.floor(f).astype(np.int64)
        i1 = np.minimum(i0 + 1, n_in - 1)
        return i0, i1, f - i0
    y0, y1, fy = taps(a.shape[2], oh)
    x0, x1, fx = taps(a.shape[3], ow)
    a = a.astype(np.float64)
    rows = a[:, :, :, x0] * (1 - fx) + a[:, :, :, x1] * fx
    return (rows[:, :, y0, :] * (1 - fy)[:, None] + rows[:, :, y1, :] * fy[:, None]).astype(np.float32)


def walk(layers, x, conv_fn, want=None, on_conv=None, upsample_fn=None, detect_fn=None):
    """Run the graph on host arrays. conv_fn(name, geometry, input_array) -> output array (fp32 NCHW, or int8 NCHW for
    int8_scale_term > 100). upsample_fn(array, oh, ow, scale, packed_rule) -> array does the bilinear Upsample layers
    (default: the float64 approximation above). Returns {blob name: array} for the names in `want` (default: the last
    layer's output)."""
    geo = conv_geometry(layers)
    blobs = {}
    for l in layers:
        t = l["type"]
        ins = [s.strip() for s in str(l.get("input", "")).split(",") if s.strip()]
        out = l["output"]
        if t == "Input":
            blobs[out] = x
        elif t == "Convolution":
            if on_conv:
                on_conv(l["name"], geo[l["name"]], blobs[ins[0]])
            blobs[out] = conv_fn(l["name"], geo[l["name"]], blobs[ins[0]])
        elif t == "MaxPool":
            a = blobs[ins[0]]
            k, s, p = int(l["kernel_h"]), int(l["stride_h"]), int(l["padding_h"])
            # the reference packs fp32 blobs with C % 4 == 0 and its packed 3x3 s2 kernels pad with zeros
            blobs[out] = maxpool_nchw(a, k, s, p, pad_zero=(a.shape[1] % 4 == 0 and k == 3 and s == 2))
        elif t == "Concat":
            blobs[out] = np.concatenate([blobs[i] for i in ins], axis=1)
        elif t == "Crop":
            blobs[out] = np.ascontiguousarray(blobs[ins[0]][:, int(l["start"]):int(l["end"])])
        elif t == "ChannelShuffle":
            a = blobs[ins[0]]
            g = int(l["groups"])
            n, c, h, w = a.shape
            blobs[out] = np.ascontiguousarray(a.reshape(n, g, c // g, h, w).transpose(0, 2, 1, 3, 4).reshape(n, c, h, w))
        elif t == "ShortCut":
            blobs[out] = blobs[ins[0]] + blobs[ins[1]]
        elif t == "NanodetPlusDetectionOutput":
            if detect_fn is None:
                raise ValueError("walk needs detect_fn(heads, strides, prob_threshold, nms_threshold) for the detection layer")
            strides = [int(v) for v in str(l.get("stride", "8, 16, 32, 64")).split(",")]
            blobs[out] = detect_fn([blobs[i] for i in ins], strides, float(l.get("prob_threshold", 0.4)), float(l.get("nms_threshold", 0.5)))
        elif t == "Upsample":
            a = blobs[ins[0]]
            if l.get("upsample_mode") != "bilinear" or str(l.get("align_corner", "false")) != "false":
                raise ValueError("only bilinear Upsample with align_corner=false is handled")
            f = float(l.get("stride", 1.0))
            # the reference resizes packed blobs (C % 4 == 0) and plain blobs with different rounding
            blobs[out] = (upsample_fn or upsample_bilinear_approx)(np.ascontiguousarray(a), int(a.shape[2] * f), int(a.shape[3] * f), f,
                                                                   1 if a.shape[1] % 4 == 0 else 0)
        elif t in ("Relu", "LRelu", "Relu6"):
            a = blobs[ins[0]]
            blobs[out] = {"Relu": lambda v: np.maximum(v, 0), "Relu6": lambda v: np.clip(v, 0, 6),
                          "LRelu": lambda v: np.where(v < 0, v * np.float32(l.get("alpha", 0.1)), v)}[t](a).astype(np.float32)
        else:
            raise ValueError(f"layer type {t} not handled")
    names = want or [layers[-1]["output"]]
    return {k: blobs[k] for k in names}


def calibrate(layers, params, x, conv_f32_fn, upsample_fn=None):
    """Fill in_scales / out_scales from one sample batch x (fp32 NCHW): 127 / max|blob| per tensor, walking the graph in
    order. conv_f32_fn(name, geometry, params_of_layer, input_array, as_float) runs one layer; with as_float=True it must
    return the layer's fp32 output even for a requantizing layer (int8_scale_term - 100), which gives the range its int8
    output scale is taken from; the consumer of an int8 blob then uses that same scale as its input scale."""
    scale_of_int8_blob = {}

    def conv_fn(name, g, a):
        p = params[name]
        n_s = g["groups"] if g["groups"] > 1 else 1
        if a.dtype == np.int8:
            s_in = scale_of_int8_blob[g["input"]]
        else:
            s_in = np.float32(127.0) / np.float32(max(float(np.abs(a).max()), 1e-6))
        p["in_scales"] = np.full((n_s,), s_in, np.float32)
        if g["term"] > 100:
            y = conv_f32_fn(name, g, p, a, True)
            s_out = np.float32(127.0) / np.float32(max(float(np.abs(y).max()), 1e-6))
            p["out_scales"] = np.full((n_s,), s_out, np.float32)
            scale_of_int8_blob[name] = s_out
        return conv_f32_fn(name, g, p, a, False)

    walk(layers, x, conv_fn, want=[l["output"] for l in layers if l["type"] == "Convolution"][-1:], upsample_fn=upsample_fn)
    return params
