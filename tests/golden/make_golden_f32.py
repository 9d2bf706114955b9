"""Freeze outputs of the compiled reference's fp32 ConvolutionLayer (int8_scale_term == 0) as a golden fixture.

Run where `make -C oracle ref` has been done (it needs the reference sources):

    python tests/golden/make_golden_f32.py

Writes tests/golden/conv_f32_small.npz: for every case of f32_cases() the seeded input, weights and bias, and the
reference's output (packed path, its default; the plain path where out_channels % 4 != 0, which the packed one refuses). The reference's fp32 kernels are built with -Ofast: they sum in their own
vector order with contractions, so these outputs pin a tolerance, not bits; the fixture also stores, per case, sum |w*x| + |b|
per output element computed in float64, which is what the tolerance is stated against.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))
from support import GOLDEN_DIR, ConvDesc, _p, load_ref  # noqa: E402


def f32_cases():
    """(name, cin, cout, k, stride, pad, groups, act, slope, bias, n, h, w, lo, hi)"""
    return [
        ("stem_3_24_s2_lrelu", 3, 24, 3, 2, 1, 1, 2, 0.1, 1, 2, 40, 40, 0.0, 1.0),   # the mixed model's first layer
        ("stem_3_20_s2_relu", 3, 20, 3, 2, 1, 1, 1, 0.0, 1, 1, 33, 37, 0.0, 1.0),    # out_channels % 4 == 0 only
        ("stem_3_8_s1_relu6_nobias", 3, 8, 3, 1, 1, 1, 3, 0.0, 0, 1, 17, 19, -1.0, 1.0),
        ("pw_16_32", 16, 32, 1, 1, 0, 1, 0, 0.0, 1, 1, 12, 12, -1.0, 1.0),
        ("dw3x3_24", 24, 24, 3, 1, 1, 24, 1, 0.0, 1, 1, 14, 14, -1.0, 1.0),
        ("dw5x5s2_16", 16, 16, 5, 2, 2, 16, 0, 0.0, 1, 1, 15, 15, -1.0, 1.0),
    ]


def make_case(c):
    name, cin, cout, k, stride, pad, groups, act, slope, bias_term, n, h, w, lo, hi = c
    rng = np.random.default_rng(sum(map(ord, name)))
    x = rng.uniform(lo, hi, size=(n, cin, h, w)).astype(np.float32)
    wt = rng.normal(0.0, 0.2, size=(cout, cin // groups, k, k)).astype(np.float32)
    b = rng.normal(0.0, 0.1, size=(cout,)).astype(np.float32)
    return x, wt, b


def conv_f64(x, wt, b, stride, pad, groups, bias_term):
    """(sum, sum of magnitudes) in float64: the exact value up to double rounding, and the scale rounding errors grow with."""
    n, cin, h, w = x.shape
    cout, cg, k, _ = wt.shape
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    xp = np.zeros((n, cin, h + 2 * pad, w + 2 * pad), np.float64)
    xp[:, :, pad:pad + h, pad:pad + w] = x
    y = np.zeros((n, cout, oh, ow), np.float64)
    mag = np.zeros_like(y)
    og = cout // groups
    for o in range(cout):
        g = o // og
        for c in range(cg):
            ci = g * cg + c
            for ky in range(k):
                for kx in range(k):
                    t = wt[o, c, ky, kx].astype(np.float64) * xp[:, ci, ky:ky + stride * oh:stride, kx:kx + stride * ow:stride][:, :oh, :ow]
                    y[:, o] += t
                    mag[:, o] += np.abs(t)
        if bias_term:
            y[:, o] += float(b[o])
            mag[:, o] += abs(float(b[o]))
    return y, mag


def main():
    ref = load_ref()
    ref.ref_conv_f32_forward.restype = C.c_int
    out = {}
    for c in f32_cases():
        name, cin, cout, k, stride, pad, groups, act, slope, bias_term, n, h, w, lo, hi = c
        x, wt, b = make_case(c)
        d = ConvDesc(cin, cout, k, k, stride, stride, pad, pad, 1, 1, groups, bias_term, 0, act, slope)
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = np.empty((n, cout, oh, ow), np.float32)
        packed = 1 if cout % 4 == 0 else 0  # the reference's packed backend has no kernel for other widths
        rc = ref.ref_conv_f32_forward(C.byref(d), _p(wt, C.c_float), _p(b, C.c_float), _p(x, C.c_float), n, h, w, packed, _p(y, C.c_float))
        assert rc == 0, (name, ref.ref_last_error())
        exact, mag = conv_f64(x, wt, b, stride, pad, groups, bias_term)
        out[f"{name}/x"], out[f"{name}/w"], out[f"{name}/b"], out[f"{name}/y"] = x, wt, b, y
        out[f"{name}/mag"] = mag.astype(np.float32)
        act_f = {0: lambda v: v, 1: lambda v: np.maximum(v, 0), 2: lambda v: np.where(v > 0, v, v * np.float64(np.float32(slope))), 3: lambda v: np.clip(v, 0, 6)}[act]
        err = np.abs(y.astype(np.float64) - act_f(exact)) / (mag * 2.0 ** -23 + 1e-30)
        print(f"{name}: reference vs float64: max {err.max():.2f} ulp of sum|w*x|+|b|")
    np.savez_compressed(GOLDEN_DIR / "conv_f32_small.npz", **out)
    print("conv_f32_small.npz", (GOLDEN_DIR / "conv_f32_small.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
