"""The fp32 ConvolutionLayer (int8_scale_term == 0), which a "mixed" quantized model keeps for its first convolution.

The reference's fp32 kernels are built with -Ofast and sum in their own vector order, so the contract is a tolerance, stated
against the magnitude sum |w*x| + |b| of each output: TOL_ULP units in the last place of that magnitude. CPU tests pin the
frozen reference outputs (tests/golden/conv_f32_small.npz, made by tests/golden/make_golden_f32.py) against a float64
evaluation and, where the compiled reference is present, against the reference run live; the GPU tests hold the library's
kernel to the same fixture, through the C-ABI and through a Net whose first layer is fp32.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

from support import GOLDEN_DIR, ConvDesc, _p, have_ref, load_ref

sys.path.insert(0, str(GOLDEN_DIR))
from make_golden_f32 import conv_f64, f32_cases, make_case  # noqa: E402

TOL_ULP = 8.0  # |ours - reference| <= TOL_ULP * 2^-23 * (sum |w*x| + |b|); the reference itself lies within 2 of float64
GOLD = np.load(GOLDEN_DIR / "conv_f32_small.npz")


def activation(v, act, slope):
    return {0: lambda a: a, 1: lambda a: np.maximum(a, 0), 2: lambda a: np.where(a > 0, a, a * np.float64(np.float32(slope))),
            3: lambda a: np.clip(a, 0, 6)}[act](v)


@pytest.mark.parametrize("case", f32_cases(), ids=lambda c: c[0])
def test_fixture_is_what_the_generator_makes_and_close_to_float64(case):
    name, cin, cout, k, stride, pad, groups, act, slope, bias_term, n, h, w, lo, hi = case
    x, wt, b = make_case(case)
    assert np.array_equal(x, GOLD[f"{name}/x"]) and np.array_equal(wt, GOLD[f"{name}/w"]) and np.array_equal(b, GOLD[f"{name}/b"])
    exact, mag = conv_f64(x, wt, b, stride, pad, groups, bias_term)
    err = np.abs(GOLD[f"{name}/y"].astype(np.float64) - activation(exact, act, slope)) / (mag * 2.0 ** -23 + 1e-30)
    assert err.max() <= 2.0, f"the frozen reference output lies {err.max():.2f} ulp from float64"


@pytest.mark.skipif(not have_ref(), reason="compiled reference not present")
@pytest.mark.parametrize("case", f32_cases(), ids=lambda c: c[0])
def test_fixture_equals_the_reference_run_live(case):
    name, cin, cout, k, stride, pad, groups, act, slope, bias_term, n, h, w, lo, hi = case
    ref = load_ref()
    ref.ref_conv_f32_forward.restype = C.c_int
    x, wt, b = make_case(case)
    d = ConvDesc(cin, cout, k, k, stride, stride, pad, pad, 1, 1, groups, bias_term, 0, act, slope)
    y = np.empty_like(GOLD[f"{name}/y"])
    assert ref.ref_conv_f32_forward(C.byref(d), _p(wt, C.c_float), _p(b, C.c_float), _p(x, C.c_float), n, h, w, 1, _p(y, C.c_float)) == 0
    assert np.array_equal(y.view(np.int32), GOLD[f"{name}/y"].view(np.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("case", f32_cases(), ids=lambda c: c[0])
def test_gpu_fp32_layer_within_tolerance_of_the_reference(case):
    from tensor_b200 import ConvF32, Context
    name, cin, cout, k, stride, pad, groups, act, slope, bias_term, n, h, w, lo, hi = case
    x, wt, b, want, mag = (GOLD[f"{name}/{t}"] for t in ("x", "w", "b", "y", "mag"))
    with Context(0) as ctx:
        layer = ConvF32(ctx, cin=cin, cout=cout, kh=k, kw=k, sh=stride, sw=stride, ph=pad, pw=pad, groups=groups, act_type=act,
                        act_param0=slope, weight=wt, bias=b if bias_term else None)
        got = layer.forward_host(x)
        layer.close()
    assert got.shape == want.shape
    err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / (mag.astype(np.float64) * 2.0 ** -23 + 1e-30)
    assert err.max() <= TOL_ULP, f"{err.max():.2f} ulp of sum|w*x|+|b| from the reference"


@pytest.mark.gpu
def test_gpu_net_with_fp32_first_layer():
    """A ShuffleNetV2-shaped graph whose first convolution is fp32, as in the reference's "mixed" int8 model: the fp32 blob is
    within tolerance of float64, and everything behind it equals the CPU checker fed with that same blob, bit for bit."""
    from graph_support import build_net, oracle_conv, oracle_conv_for_calibration
    from graph_walk import calibrate, walk
    from tensor_b200 import graphs
    L = graphs.shufflenetv2_layers(64, 64, batch=2, act="LRelu")
    assert L[1]["name"] == "conv1"
    L[1]["int8_scale_term"] = 0
    rng = np.random.default_rng(64)
    x = rng.uniform(0, 1, size=(2, 3, 64, 64)).astype(np.float32)
    w1 = rng.normal(0, 0.2, size=(24, 3, 3, 3)).astype(np.float32)
    b1 = rng.normal(0, 0.1, size=(24,)).astype(np.float32)
    exact, mag = conv_f64(x, w1, b1, 2, 1, 1, 1)
    conv1_f64 = activation(exact, 2, 0.1)
    params = graphs.make_params(L)
    int8_params = {k: v for k, v in params.items() if k != "conv1"}

    def first_layer_then(fn, conv1_blob):
        return lambda name, g, *a: conv1_blob(*a) if name == "conv1" else fn(name, g, *a)

    calibrate(L, params, x[:1], first_layer_then(oracle_conv_for_calibration, lambda p, a, as_float: conv1_f64[:a.shape[0]].astype(np.float32)))
    net = build_net(L, int8_params, options={"fuse_first_layer_pool": 1})
    net.set_conv_params_f32("conv1", w1, b1)
    conv1 = net.forward("data", x, ["conv1"])[0]
    err = np.abs(conv1.astype(np.float64) - conv1_f64) / (mag * 2.0 ** -23 + 1e-30)
    assert err.max() <= TOL_ULP
    probes = ["pool1", "s2b0_shuf", "s3b0_shuf", "conv5"]
    want = walk(L, x, first_layer_then(oracle_conv(params), lambda a: conv1), want=probes)
    got = net.forward("data", x, probes)
    for name, g in zip(probes, got):
        assert np.array_equal(g.view(np.int32), want[name].view(np.int32)), f"blob {name} differs"
    net.close()
