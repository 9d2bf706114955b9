"""Benchmark graphs as lists of the reference's LayerOption dictionaries, plus seeded parameters.

`shufflenetv2_layers` writes ShuffleNetV2-1.0x in the same layer vocabulary and wiring as the reference's
own int8 graph (benchmark/nanodet-plus-m-1.5x_416_int8_fused.otter: stem convolution -> MaxPool -> stages of
[Crop, 1x1 (int8 out) -> depthwise 3x3 (int8 out) -> 1x1 (fp32 out), Concat, ChannelShuffle]), so the list can be
fed to `Net.add_layer` here or written out as a .otter file for the reference.

Only descriptions live here: layer lists, shape inference and seeded parameters. Nothing in this module executes a graph.
"""
from __future__ import annotations

import numpy as np

ACT_CODE = {"": 0, "Relu": 1, "LRelu": 2, "Relu6": 3}


def _conv(name, inp, cout, k, stride, pad, term, act="", groups=1):
    d = dict(type="Convolution", name=name, input=inp, output=name, out_channels=cout, kernel_h=k, kernel_w=k, stride_h=stride,
             stride_w=stride, padding_h=pad, padding_w=pad, dilation_h=1, dilation_w=1, int8_scale_term=term, bias_term="true")
    if groups != 1:
        d["groups"] = groups
    if act:
        d["activation"] = act
        if act == "LRelu":
            d["activation_params"] = "0.100000"
    return d


def shufflenetv2_layers(height=320, width=320, batch=1, stage_repeats=(4, 8, 4), stage_channels=(116, 232, 464), stem=24, last=1024,
                        act="Relu"):
    """ShuffleNetV2-1.0x backbone (conv1 3x3 s2 24, maxpool, stages [4,8,4] x [116,232,464], conv5 1x1 1024), quantized
    the way the reference's int8 graphs are: int8 only flows conv -> conv inside a branch, fp32 everywhere else."""
    L = [dict(type="Input", name="data", output="data", batchsize=batch, channel=3, height=height, width=width)]
    L.append(_conv("conv1", "data", stem, 3, 2, 1, 2, act))
    L.append(dict(type="MaxPool", name="pool1", input="conv1", output="pool1", kernel_h=3, kernel_w=3, stride_h=2, stride_w=2,
                  padding_h=1, padding_w=1))
    prev, cin = "pool1", stem
    for si, (rep, cout) in enumerate(zip(stage_repeats, stage_channels)):
        half = cout // 2
        s = f"s{si + 2}"
        # down-sampling unit: both branches see the whole input
        L.append(_conv(f"{s}b0_l_dw", prev, cin, 3, 2, 1, 101, "", groups=cin))
        L.append(_conv(f"{s}b0_l_pw", f"{s}b0_l_dw", half, 1, 1, 0, 2, act))
        L.append(_conv(f"{s}b0_r_pw1", prev, half, 1, 1, 0, 102, act))
        L.append(_conv(f"{s}b0_r_dw", f"{s}b0_r_pw1", half, 3, 2, 1, 101, "", groups=half))
        L.append(_conv(f"{s}b0_r_pw2", f"{s}b0_r_dw", half, 1, 1, 0, 2, act))
        L.append(dict(type="Concat", name=f"{s}b0_cat", input=f"{s}b0_l_pw, {s}b0_r_pw2", output=f"{s}b0_cat", axis=1))
        L.append(dict(type="ChannelShuffle", name=f"{s}b0_shuf", input=f"{s}b0_cat", output=f"{s}b0_shuf", groups=2))
        prev = f"{s}b0_shuf"
        for bi in range(1, rep):
            b = f"{s}b{bi}"
            L.append(dict(type="Crop", name=f"{b}_keep", input=prev, output=f"{b}_keep", start=0, end=half, axis=1))
            L.append(dict(type="Crop", name=f"{b}_work", input=prev, output=f"{b}_work", start=half, end=cout, axis=1))
            L.append(_conv(f"{b}_pw1", f"{b}_work", half, 1, 1, 0, 102, act))
            L.append(_conv(f"{b}_dw", f"{b}_pw1", half, 3, 1, 1, 101, "", groups=half))
            L.append(_conv(f"{b}_pw2", f"{b}_dw", half, 1, 1, 0, 2, act))
            L.append(dict(type="Concat", name=f"{b}_cat", input=f"{b}_keep, {b}_pw2", output=f"{b}_cat", axis=1))
            L.append(dict(type="ChannelShuffle", name=f"{b}_shuf", input=f"{b}_cat", output=f"{b}_shuf", groups=2))
            prev = f"{b}_shuf"
        cin = cout
    if last:
        L.append(_conv("conv5", prev, last, 1, 1, 0, 2, act))
    return L


def nanodet_plus_layers(height=320, width=320, batch=1, neck=96, classes=80, reg_max=7, stage_repeats=(4, 8, 4),
                        stage_channels=(116, 232, 464), stem=24, act="LRelu", detect=False):
    """A NanoDet-Plus-style int8 detector in the wiring of the reference's own graph
    (benchmark/nanodet-plus-m-1.5x_416_int8_fused.otter, layers conv_56 ... conv_110) on the ShuffleNetV2-1.0x backbone:
    three 1x1 reductions to `neck` channels; a Ghost-PAN neck (top-down with bilinear x2 Upsample + Concat, bottom-up with
    depthwise 5x5 stride-2 + 1x1, each merge a Ghost block = two ghost modules [1x1 -> depthwise 3x3, Concat] plus a
    depthwise 5x5 -> 1x1 shortcut, added by ShortCut); an extra stride-64 level; and per level a head of
    2 x [depthwise 5x5 -> 1x1] and a 1x1 to classes + 4*(reg_max+1) channels. Outputs: head8, head16, head32, head64;
    with detect=True also the NanodetPlusDetectionOutput layer that decodes them into boxes."""
    L = shufflenetv2_layers(height, width, batch, stage_repeats, stage_channels, stem, last=0, act=act)
    half = neck // 2
    feats = [f"s{si + 2}b{rep - 1}_shuf" for si, rep in enumerate(stage_repeats)]
    for tag, src in zip(("r8", "r16", "r32"), feats):
        L.append(_conv(tag, src, neck, 1, 1, 0, 2, act))

    def cat(name, a, b):
        L.append(dict(type="Concat", name=name, input=f"{a}, {b}", output=name, axis=1))
        return name

    def ghost_block(tag, src):  # src has 2*neck channels; result has neck
        L.append(_conv(f"{tag}_g1pw", src, half, 1, 1, 0, 2, act))
        L.append(_conv(f"{tag}_g1dw", f"{tag}_g1pw", half, 3, 1, 1, 1, act, groups=half))
        cat(f"{tag}_g1", f"{tag}_g1pw", f"{tag}_g1dw")
        L.append(_conv(f"{tag}_g2pw", f"{tag}_g1", half, 1, 1, 0, 2))
        L.append(_conv(f"{tag}_g2dw", f"{tag}_g2pw", half, 3, 1, 1, 1, "", groups=half))
        cat(f"{tag}_g2", f"{tag}_g2pw", f"{tag}_g2dw")
        L.append(_conv(f"{tag}_scdw", src, 2 * neck, 5, 1, 2, 101, "", groups=2 * neck))
        L.append(_conv(f"{tag}_scpw", f"{tag}_scdw", neck, 1, 1, 0, 2))
        L.append(dict(type="ShortCut", name=tag, input=f"{tag}_g2, {tag}_scpw", output=tag))
        return tag

    def up(name, src):
        L.append(dict(type="Upsample", name=name, input=src, output=name, upsample_mode="bilinear", align_corner="false", stride="2.000000"))
        return name

    def down(tag, src):
        L.append(_conv(f"{tag}_dw", src, neck, 5, 2, 2, 101, act, groups=neck))
        L.append(_conv(tag, f"{tag}_dw", neck, 1, 1, 0, 2, act))
        return tag

    td16 = ghost_block("td16", cat("td16_in", up("up32", "r32"), "r16"))
    td8 = ghost_block("td8", cat("td8_in", up("up16", td16), "r8"))
    bu16 = ghost_block("bu16", cat("bu16_in", down("dn8", td8), td16))
    bu32 = ghost_block("bu32", cat("bu32_in", down("dn16", bu16), "r32"))
    L.append(dict(type="ShortCut", name="p64", input=f"{down('ex_a', 'r32')}, {down('ex_b', bu32)}", output="p64"))
    for tag, src in zip(("head8", "head16", "head32", "head64"), (td8, bu16, bu32, "p64")):
        L.append(_conv(f"{tag}_dw1", src, neck, 5, 1, 2, 101, act, groups=neck))
        L.append(_conv(f"{tag}_pw1", f"{tag}_dw1", neck, 1, 1, 0, 102, act))
        L.append(_conv(f"{tag}_dw2", f"{tag}_pw1", neck, 5, 1, 2, 101, act, groups=neck))
        L.append(_conv(f"{tag}_pw2", f"{tag}_dw2", neck, 1, 1, 0, 102, act))
        L.append(_conv(tag, f"{tag}_pw2", classes + 4 * (reg_max + 1), 1, 1, 0, 2))
    if detect:  # the decode layer at the end of the reference's graph (its last layer, "nanodet")
        L.append(dict(type="NanodetPlusDetectionOutput", name="nanodet", input=", ".join(NANODET_OUTPUTS), output="nanodet",
                      prob_threshold="0.400000", nms_threshold="0.500000", stride="8, 16, 32, 64"))
    return L


NANODET_OUTPUTS = ("head8", "head16", "head32", "head64")


def shipped_nanodet_plus_layers(batch=1, mixed=False, detect=True):
    """The detector the reference ships as benchmark/nanodet-plus-m-1.5x_416_int8_fused.otter (mixed=True:
    ..._int8_mixed.otter, whose first convolution stays fp32, int8_scale_term 0): ShuffleNetV2-1.5x widths, 128 neck channels,
    416x416 input. Same layers in the same order with the same parameters and wiring as those files; only names differ."""
    L = nanodet_plus_layers(416, 416, batch=batch, neck=128, stage_channels=(176, 352, 704), detect=detect)
    if mixed:
        conv1 = next(l for l in L if l["type"] == "Convolution")
        conv1["int8_scale_term"] = 0
    return L


def to_otter_text(layers, name="generated by tensor_b200.graphs") -> str:
    """The layer list as a `.otter` text graph, in the layout of the reference's own files: structural keys first,
    the layer's parameters in a nested Param block."""
    structural = ("type", "name", "input", "output", "activation")
    out = [f'name: "{name}"']
    for l in layers:
        out.append(f'{l["type"]} {{')
        for k in ("activation", "name", "input", "output"):
            if k in l:
                v = str(l[k])
                out.append(f'    {k}: "{v}"' if ("," in v or " " in v) else f"    {k}: {v}")
        params = [(k, v) for k, v in l.items() if k not in structural]
        if params:
            out.append("    Param {")
            out += [f'        {k}: "{v}"' if ("," in str(v) or " " in str(v)) else f"        {k}: {v}" for k, v in params]
            out.append("    }")
        out.append("}")
    return "\n".join(out) + "\n"


def conv_geometry(layers):
    """name -> dict(cin, cout, k, stride, pad, groups, term, act) for every Convolution, with cin from shape inference."""
    chans = {}
    geo = {}
    for l in layers:
        t = l["type"]
        ins = [s.strip() for s in str(l.get("input", "")).split(",") if s.strip()]
        if t == "Input":
            chans[l["output"]] = int(l["channel"])
        elif t == "Convolution":
            cin = chans[ins[0]]
            geo[l["name"]] = dict(cin=cin, cout=int(l["out_channels"]), k=int(l["kernel_h"]), stride=int(l["stride_h"]), pad=int(l["padding_h"]),
                                  groups=int(l.get("groups", 1)), term=int(l["int8_scale_term"]), act=ACT_CODE[l.get("activation", "")],
                                  act_param0=0.1 if l.get("activation") == "LRelu" else 0.0, input=ins[0])
            chans[l["output"]] = int(l["out_channels"])
        elif t == "Concat":
            chans[l["output"]] = sum(chans[i] for i in ins)
        elif t == "Crop":
            chans[l["output"]] = int(l["end"]) - int(l["start"])
        else:
            chans[l["output"]] = chans[ins[0]]
    return geo


def conv_input_hw(layers, height, width):
    """name -> (h, w) of the blob each Convolution reads, and total multiply-accumulates per image."""
    hw, out, macs = {}, {}, 0
    geo = conv_geometry(layers)
    for l in layers:
        ins = [s.strip() for s in str(l.get("input", "")).split(",") if s.strip()]
        if l["type"] == "Input":
            hw[l["output"]] = (height, width)
            continue
        h, w = hw[ins[0]]
        if l["type"] in ("Convolution", "MaxPool"):
            k, s_, p_ = int(l["kernel_h"]), int(l["stride_h"]), int(l["padding_h"])
            oh, ow = (h + 2 * p_ - k) // s_ + 1, (w + 2 * p_ - k) // s_ + 1
            hw[l["output"]] = (oh, ow)
            if l["type"] == "Convolution":
                g = geo[l["name"]]
                out[l["name"]] = (h, w)
                macs += oh * ow * g["cout"] * (g["cin"] // g["groups"]) * k * k
        elif l["type"] == "Upsample":
            f = float(l.get("stride", 1.0))
            hw[l["output"]] = (int(h * f), int(w * f))
        else:
            hw[l["output"]] = (h, w)
    return out, macs


def make_params(layers, seed=0x0771E5):
    """Seeded weights per Convolution: N(0, 0.05) (depthwise N(0, 0.1)) quantized per output channel, bias N(0, 0.01).
    Activation scales are placeholders until `calibrate` fills them."""
    rng = np.random.default_rng(seed)
    params = {}
    for name, g in conv_geometry(layers).items():
        dw = g["groups"] > 1
        wf = rng.normal(0.0, 0.1 if dw else 0.05, size=(g["cout"], g["cin"] // g["groups"], g["k"], g["k"])).astype(np.float32)
        amax = np.abs(wf).reshape(g["cout"], -1).max(axis=1)
        amax[amax == 0] = 1.0
        w_scales = (np.float32(127.0) / amax).astype(np.float32)
        params[name] = dict(weight=np.clip(np.rint(wf * w_scales[:, None, None, None]), -127, 127).astype(np.int8),
                            bias=rng.normal(0.0, 0.01, size=(g["cout"],)).astype(np.float32), w_scales=w_scales,
                            in_scales=np.ones((g["groups"] if dw else 1,), np.float32),
                            out_scales=np.ones((g["groups"] if dw else 1,), np.float32) if g["term"] > 100 else None)
    return params
