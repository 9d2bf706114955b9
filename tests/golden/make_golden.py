"""Freeze outputs of the compiled reference (oracle/_ref/libotter_ref.so) as golden fixtures.

Run in a checkout where `make -C oracle ref` has been done (it needs the reference sources):

    python tests/golden/make_golden.py

Writes tests/golden/conv_int8_small.npz: for every case of tests/cases.py the seeded inputs' checksum,
SHA-256 digests of the int8 activations the layer convolved and of the exact s32 accumulators, and the
final output in full, as produced
by the reference's own code on the path named in the case list ("packed", "unpacked"). Cases marked
"port" cannot be run by the reference at all (it corrupts its heap on them); for those the s32
accumulators come from the C restatement and the epilogue from the reference's own
requantize/dequantize functions applied to them.
Also writes tests/golden/epilogue_adversarial.npz: accumulators and scales picked so that a fused
multiply-add and a separate multiply+add disagree, and values on both rounding rules' tie points,
with the reference's answers.
Also writes tests/golden/net_nanodet_wide_small.npz (the same for the detector graph of graph_support.wide_nanodet_case) and
tests/golden/net_shufflenet_wide_small.npz: blobs of a whole ShuffleNetV2-shaped graph (channel widths all
multiples of 8) run through the reference's own Net (load_otter -> Extractor), one 64x64 image.
"""
import ctypes as C
import hashlib
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))
from cases import small_cases  # noqa: E402
from support import (GOLDEN_DIR, _p, load_port, load_ref, rounding_for, run_port,  # noqa: E402
                     run_ref)


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def ref_epilogue_on_port_acc(case, acc, packed):
    """Reference epilogue functions applied to accumulators the reference cannot produce itself."""
    ref, port = load_ref(), load_port()
    scale_in = np.empty((case.cout,), np.float32)
    port.orc_scale_in(_p(case.w_scales, C.c_float), C.c_int(case.cout), C.c_float(float(case.in_scales[0])), _p(scale_in, C.c_float))
    n, c, oh, ow = acc.shape
    outs = []
    for i in range(n):
        a = np.ascontiguousarray(acc[i])
        nb = case.cout if case.bias_term else 0
        if case.requant:
            y = np.empty((c, oh, ow), np.int8)
            rc = ref.ref_requantize(_p(a, C.c_int32), c, oh, ow, _p(scale_in, C.c_float), c, _p(case.out_scales, C.c_float),
                                    int(case.out_scales.size), _p(case.bias, C.c_float), nb, case.act_type,
                                    C.c_float(case.act_param0), packed, _p(y, C.c_int8))
        else:
            y = np.empty((c, oh, ow), np.float32)
            rc = ref.ref_dequantize(_p(a, C.c_int32), c, oh, ow, _p(scale_in, C.c_float), c, _p(case.bias, C.c_float), nb, packed,
                                    _p(y, C.c_float))
            assert case.act_type == 0
        assert rc == 0, ref.ref_last_error()
        outs.append(y)
    return np.stack(outs)


def adversarial_epilogue(rng):
    """Accumulator / scale / bias triples where fma(acc,s,b) != acc*s+b, plus rounding ties."""
    c, hw = 64, 384
    acc = rng.integers(-200000, 200001, size=(c, 1, hw), dtype=np.int32)
    scale_in = rng.uniform(1e-5, 3e-3, size=c).astype(np.float32)
    bias = rng.normal(0, 0.3, size=c).astype(np.float32)
    scale_out = np.array([rng.uniform(5.0, 60.0)], np.float32)
    return acc, scale_in, bias, scale_out


def main():
    ref = load_ref()
    out = {}
    for case, path in small_cases():
        case.make()
        packed = path.startswith("packed")
        if path.startswith("port"):
            got = run_port(case, rounding_for(path))
            got["y"] = ref_epilogue_on_port_acc(case, got["acc"], 1 if path == "port_packed_epilogue" else 0)
        else:
            got = run_ref(case, packed)
        k = case.name
        out[k + "/inputs_sha256"] = np.frombuffer(digest(case.weight, case.bias, case.w_scales, case.in_scales, case.out_scales,
                                                         case.x_f32, case.x_s8).encode(), dtype=np.uint8)
        out[k + "/xq_sha256"] = np.frombuffer(digest(got["xq"]).encode(), dtype=np.uint8)
        out[k + "/acc_sha256"] = np.frombuffer(digest(got["acc"]).encode(), dtype=np.uint8)
        out[k + "/y"] = got["y"]
    np.savez_compressed(GOLDEN_DIR / "conv_int8_small.npz", **out)

    rng = np.random.default_rng(20240531)
    acc, scale_in, bias, scale_out = adversarial_epilogue(rng)
    c, _, hw = acc.shape
    adv = {"acc": acc, "scale_in": scale_in, "bias": bias, "scale_out": scale_out}
    for packed in (1, 0):
        tag = "packed" if packed else "unpacked"
        y = np.empty((c, 1, hw), np.float32)
        assert ref.ref_dequantize(_p(acc, C.c_int32), c, 1, hw, _p(scale_in, C.c_float), c, _p(bias, C.c_float), c, packed, _p(y, C.c_float)) == 0
        adv[f"dequant_{tag}"] = y
        for act, slope in ((0, 0.0), (1, 0.0), (2, 0.1), (3, 0.0)):
            q = np.empty((c, 1, hw), np.int8)
            assert ref.ref_requantize(_p(acc, C.c_int32), c, 1, hw, _p(scale_in, C.c_float), c, _p(scale_out, C.c_float), 1,
                                      _p(bias, C.c_float), c, act, C.c_float(slope), packed, _p(q, C.c_int8)) == 0
            adv[f"requant_act{act}_{tag}"] = q
    # quantize ties: x*scale lands on k+0.5 and on the one float (0.49999997) where the two rules differ
    ties = np.concatenate([np.arange(-130, 131, dtype=np.float32) + np.float32(0.5),
                           np.array([0.49999997, -0.49999997, 0.5, -0.5, 126.5, 127.49, 127.5, 1e9, -1e9, 0.0, -0.0], np.float32)])
    ties = np.resize(ties, (8, 4, 68)).astype(np.float32).copy()
    adv["ties"] = ties
    one = np.ones((1,), np.float32)
    for packed in (1, 0):
        q = np.empty(ties.shape, np.int8)
        assert ref.ref_quantize(_p(ties, C.c_float), 8, 4, 68, _p(one, C.c_float), 1, packed, _p(q, C.c_int8)) == 0
        adv[f"ties_q_{'packed' if packed else 'unpacked'}"] = q
    np.savez_compressed(GOLDEN_DIR / "epilogue_adversarial.npz", **adv)
    # whole graph through the reference's own Net (widths all multiples of 8)
    from graph_support import reference_net_forward, wide_shufflenet_case
    L, params, x, blobs = wide_shufflenet_case()
    got = reference_net_forward(L, params, x, blobs)
    net = {"input_sha256": np.frombuffer(digest(x, *[params[k]["weight"] for k in sorted(params)], *[params[k]["in_scales"] for k in sorted(params)]).encode(), dtype=np.uint8)}
    for b in blobs:
        net[b] = got[b]
    np.savez_compressed(GOLDEN_DIR / "net_shufflenet_wide_small.npz", **net)
    # the detector graph (backbone + Ghost-PAN neck with bilinear Upsample / ShortCut + heads) through the reference's Net
    from graph_support import wide_nanodet_case
    L, params, x, blobs = wide_nanodet_case()
    got = reference_net_forward(L, params, x, blobs)
    det = {"input_sha256": np.frombuffer(digest(x, *[params[k]["weight"] for k in sorted(params)], *[params[k]["in_scales"] for k in sorted(params)]).encode(), dtype=np.uint8)}
    for b in blobs:
        det[b] = got[b]
    # the reference's own decode of those heads (NanodetPlusDetectionOutput layer): rows {label + 1, score, x, y, w, h}
    from test_graph_oracle import ref_layer
    from tensor_b200 import graphs
    det["detections"] = ref_layer("NanodetPlusDetectionOutput", "prob_threshold=0.4;nms_threshold=0.5;stride=8, 16, 32, 64",
                                  [got[k] for k in graphs.NANODET_OUTPUTS], packed=0).reshape(-1, 6)
    np.savez_compressed(GOLDEN_DIR / "net_nanodet_wide_small.npz", **det)
    for f in ("conv_int8_small.npz", "epilogue_adversarial.npz", "net_shufflenet_wide_small.npz", "net_nanodet_wide_small.npz"):
        print(f, (GOLDEN_DIR / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
