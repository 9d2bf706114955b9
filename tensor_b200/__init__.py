"""tensor_b200 — B200 (sm_100a) int8 convolution path behind Otter's Net / Layer / ConvolutionLayer API.

The product is the native library `lib/libotter_b200.so` (CUDA kernels + C-ABI, include/otter_b200.h)
and the C++17 host mirror of the reference's operator API under `host/`. This Python package only builds
the library and binds its C-ABI with ctypes for the tests and the benchmark; it computes nothing itself
and has no CPU path: if the library is missing or no GPU is present, calls fail.
"""
from .capi import (ACT_LRELU, ACT_NONE, ACT_RELU, ACT_RELU6, F32_NCHW, KERNEL_DENSE_DIRECT, KERNEL_DENSE_UMMA,  # noqa: F401
                   KERNEL_DEPTHWISE, ROUND_ADD_HALF_TRUNC, ROUND_HALF_AWAY, S8_NHWC, S32_NHWC, ConvF32, ConvInt8, Context,
                   DwPwInt8, Net, NetGroup, OtterB200Error, UnitInt8, library, library_path, nhwc_channels, partition)
