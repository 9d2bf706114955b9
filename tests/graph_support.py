"""Graph-level checker: the benchmark graphs executed layer by layer with the CPU checkers (convolutions through the
C restatement of the reference, glue layers in numpy as validated against the compiled reference)."""
from __future__ import annotations

import numpy as np

from support import ConvCase, run_port
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


def oracle_conv_for_calibration(name, g, p, a, as_float):
    term = g["term"] - 100 if (as_float and g["term"] > 100) else g["term"]
    return run_port(_case(name, g, p, a, term), 0, want_acc=False)["y"]


def build_net(layers, params, device=0):
    from tensor_b200 import Net
    net = Net(device)
    for l in layers:
        net.add_layer(**l)
    net.compile()
    for name, p in params.items():
        net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    return net
