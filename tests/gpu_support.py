"""Helpers of the GPU parity tests: run one seeded case through the C-ABI and bring the results back in
the reference's boundary layout (NCHW) for comparison with the CPU checkers."""
from __future__ import annotations

import numpy as np

from support import ConvCase, nchw_to_nhwc_padded, nhwc_padded_to_nchw, rounding_for
from tensor_b200 import F32_NCHW, S8_NHWC, S32_NHWC, ConvInt8, Context, nhwc_channels


def make_layer(ctx: Context, case: ConvCase, rounding: int) -> ConvInt8:
    return ConvInt8(ctx, cin=case.cin, cout=case.cout, kh=case.k, kw=case.kwid, sh=case.stride, sw=case.stride, ph=case.pad,
                    pw=case.pad, dh=case.dil, dw=case.dil, groups=case.groups, bias_term=case.bias_term,
                    int8_scale_term=case.int8_scale_term, act_type=case.act_type, act_param0=case.act_param0, rounding=rounding,
                    weight=case.weight, bias=case.bias if case.bias_term else None, w_scales=case.w_scales,
                    in_scales=case.in_scales, out_scales=case.out_scales if case.requant else None)


def run_gpu(ctx: Context, case: ConvCase, rounding: int, want_acc: bool = True):
    """Returns {"acc": s32 NCHW or None, "y": final output NCHW, "kind": kernel kind}."""
    layer = make_layer(ctx, case, rounding)
    try:
        if case.s8_input:
            x, in_dtype = nchw_to_nhwc_padded(case.x_s8, nhwc_channels(case.cin)), S8_NHWC
        else:
            x, in_dtype = case.x_f32, F32_NCHW
        out = {"kind": layer.kernel_kind, "acc": None}
        if want_acc:
            acc = layer.forward_host(x, in_dtype, S32_NHWC)
            out["acc"] = nhwc_padded_to_nchw(acc, case.cout)
            out["acc_pad"] = acc[..., case.cout:]
        if case.requant:
            y = layer.forward_host(x, in_dtype, S8_NHWC)
            out["y_pad"] = y[..., case.cout:]
            out["y"] = nhwc_padded_to_nchw(y, case.cout)
        else:
            out["y"] = layer.forward_host(x, in_dtype, F32_NCHW)
        return out
    finally:
        layer.close()


def bits(a):
    return a.view(np.int32) if a.dtype == np.float32 else a
