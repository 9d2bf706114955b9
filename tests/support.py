"""Shared test harness: seeded synthetic int8-convolution cases and ctypes bindings to the two
CPU checkers (the plain-C restatement under oracle/ and, when it has been built, the compiled
reference under oracle/_ref/). Nothing in the shipped library imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
PORT_SO = ORACLE_DIR / "_build" / "libotter_oracle.so"
REF_SO = ORACLE_DIR / "_ref" / "libotter_ref.so"
GOLDEN_DIR = ROOT / "tests" / "golden"

ROUND_ADD_HALF_TRUNC = 0  # packed x86 path (the reference's default)
ROUND_HALF_AWAY = 1  # unpacked x86 path / aarch64

ACT_NONE, ACT_RELU, ACT_LRELU, ACT_RELU6 = 0, 1, 2, 3


class ConvDesc(C.Structure):
    """Mirror of orc_conv_desc / the reference driver's RefConvDesc / ott_conv_desc (same field order)."""

    _fields_ = [(k, C.c_int) for k in ("cin", "cout", "kh", "kw", "sh", "sw", "ph", "pw", "dh", "dw", "groups",
                                       "bias_term", "int8_scale_term", "act_type")] + [("act_param0", C.c_float)]


def _p(a, ty):
    return None if a is None else a.ctypes.data_as(C.POINTER(ty))


def build_port() -> Path:
    """Compile the plain-C restatement (seconds) if it is missing or stale."""
    src = ORACLE_DIR / "otter_int8_oracle.c"
    if not PORT_SO.exists() or PORT_SO.stat().st_mtime < max(src.stat().st_mtime, (ORACLE_DIR / "otter_int8_oracle.h").stat().st_mtime):
        subprocess.run(["make", "-s", "-C", str(ORACLE_DIR), "port"], check=True)
    return PORT_SO


_port = None
_ref = None


def load_port():
    global _port
    if _port is None:
        lib = C.CDLL(str(build_port()))
        lib.orc_float2int8.restype = C.c_int8
        lib.orc_float2int8.argtypes = [C.c_float, C.c_int]
        lib.orc_conv_int8_forward.restype = C.c_int
        lib.orc_max_threads.restype = C.c_int
        _port = lib
    return _port


def have_ref() -> bool:
    return REF_SO.exists()


def load_ref():
    global _ref
    if _ref is None:
        lib = C.CDLL(str(REF_SO))
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_conv_int8_forward.restype = C.c_int
        lib.ref_conv_int8_time_ms.restype = C.c_double
        lib.ref_max_threads.restype = C.c_int
        _ref = lib
    return _ref


@dataclass
class ConvCase:
    """One quantized ConvolutionLayer plus the batch it runs on. Arrays follow the reference's
    boundary layouts: weights OIHW int8, activations NCHW."""

    name: str
    cin: int
    cout: int
    k: int
    stride: int = 1
    pad: int = 0
    groups: int = 1
    n: int = 1
    h: int = 8
    w: int = 8
    bias_term: int = 1
    int8_scale_term: int = 2
    act_type: int = ACT_NONE
    act_param0: float = 0.0
    seed: int = 0
    w_std: float = 0.05
    x_lo: float = -1.0
    x_hi: float = 1.0
    s8_input: bool = False
    dil: int = 1
    kw: int | None = None  # kernel width when it differs from k (height)
    # filled by make()
    weight: np.ndarray = field(default=None, repr=False)
    bias: np.ndarray = field(default=None, repr=False)
    w_scales: np.ndarray = field(default=None, repr=False)
    in_scales: np.ndarray = field(default=None, repr=False)
    out_scales: np.ndarray = field(default=None, repr=False)
    x_f32: np.ndarray = field(default=None, repr=False)
    x_s8: np.ndarray = field(default=None, repr=False)

    @property
    def depthwise(self) -> bool:
        return self.groups == self.cin == self.cout and self.groups > 1

    @property
    def kwid(self) -> int:
        return self.k if self.kw is None else self.kw

    @property
    def oh(self) -> int:
        return (self.h + 2 * self.pad - self.dil * (self.k - 1) - 1) // self.stride + 1

    @property
    def ow(self) -> int:
        return (self.w + 2 * self.pad - self.dil * (self.kwid - 1) - 1) // self.stride + 1

    @property
    def requant(self) -> bool:
        return self.int8_scale_term > 100

    def desc(self) -> ConvDesc:
        return ConvDesc(self.cin, self.cout, self.k, self.kwid, self.stride, self.stride, self.pad, self.pad,
                        self.dil, self.dil, self.groups, self.bias_term, self.int8_scale_term, self.act_type,
                        self.act_param0)

    def make(self, dry_run: bool = True) -> "ConvCase":
        """Seeded synthetic tensors with the distributions the benchmark configurations name:
        activations uniform, weights normal quantized per output channel (scale = 127/max|w|),
        bias normal(0, 0.01), activation scale 127/max|x| per tensor, output scale from a float dry run."""
        rng = np.random.default_rng(0x0771E5 + self.seed)
        cin_g = self.cin // self.groups
        wf = rng.normal(0.0, self.w_std, size=(self.cout, cin_g, self.k, self.kwid)).astype(np.float32)
        amax = np.abs(wf).reshape(self.cout, -1).max(axis=1)
        amax[amax == 0] = 1.0
        self.w_scales = (np.float32(127.0) / amax).astype(np.float32)
        self.weight = np.clip(np.rint(wf * self.w_scales[:, None, None, None]), -127, 127).astype(np.int8)
        self.bias = rng.normal(0.0, 0.01, size=(self.cout,)).astype(np.float32)
        x = rng.uniform(self.x_lo, self.x_hi, size=(self.n, self.cin, self.h, self.w)).astype(np.float32)
        s_in = np.float32(127.0) / np.float32(max(np.abs(x).max(), 1e-6))
        # the layer keeps [groups] copies of the activation scale for depthwise (ConvolutionLayer.cpp:262-265)
        self.in_scales = np.full((self.groups if self.depthwise else 1,), s_in, dtype=np.float32)
        if self.s8_input:
            self.x_s8 = rng.integers(-127, 128, size=x.shape, dtype=np.int8)
            self.x_f32 = None
        else:
            self.x_f32 = x
            self.x_s8 = None
        if self.requant:
            # rough float dry run on a slice to pick an output scale of the right magnitude
            std = self.w_std * np.sqrt(cin_g * self.k * self.kwid / 3.0) * (127.0 if self.s8_input else 1.0) / (s_in if self.s8_input else 1.0)
            top = np.float32(max(4.0 * std, 1e-3))
            if self.act_type == ACT_RELU6:
                top = np.float32(min(top, 6.0))
            s_out = np.float32(127.0) / top
            self.out_scales = np.full((self.groups if self.depthwise else 1,), s_out, dtype=np.float32)
            if dry_run:
                # 127 / max|act(y)| of the float output the same layer gives without requantization
                import copy
                probe = copy.copy(self)
                probe.int8_scale_term = self.int8_scale_term - 100
                y = run_port(probe, want_acc=False)["y"]
                top = np.float32(max(float(np.abs(y).max()), 1e-6))
                self.out_scales[:] = np.float32(127.0) / top
        else:
            self.out_scales = np.zeros((1,), dtype=np.float32)
        return self


def _run(lib_fn, case: ConvCase, last_int_arg: int, want_acc=True):
    d = case.desc()
    n, oh, ow = case.n, case.oh, case.ow
    xq = np.empty((n, case.cin, case.h, case.w), dtype=np.int8)
    acc = np.empty((n, case.cout, oh, ow), dtype=np.int32) if want_acc else None
    y_f32 = None if case.requant else np.empty((n, case.cout, oh, ow), dtype=np.float32)
    y_s8 = np.empty((n, case.cout, oh, ow), dtype=np.int8) if case.requant else None
    rc = lib_fn(C.byref(d), _p(case.weight, C.c_int8), _p(case.bias, C.c_float), _p(case.w_scales, C.c_float),
                _p(case.in_scales, C.c_float), C.c_int(case.in_scales.size), _p(case.out_scales, C.c_float),
                C.c_int(case.out_scales.size), _p(case.x_f32, C.c_float), _p(case.x_s8, C.c_int8), C.c_int(n),
                C.c_int(case.h), C.c_int(case.w), C.c_int(last_int_arg), _p(xq, C.c_int8), _p(acc, C.c_int32),
                _p(y_f32, C.c_float), _p(y_s8, C.c_int8))
    return rc, {"xq": xq, "acc": acc, "y": y_s8 if case.requant else y_f32}


def run_port(case: ConvCase, rounding: int = ROUND_ADD_HALF_TRUNC, want_acc=True):
    rc, out = _run(load_port().orc_conv_int8_forward, case, rounding, want_acc)
    assert rc == 0, f"oracle port failed rc={rc}"
    return out


def run_ref(case: ConvCase, packed: bool = True, want_acc=True):
    lib = load_ref()
    rc, out = _run(lib.ref_conv_int8_forward, case, 1 if packed else 0, want_acc)
    if rc != 0:
        raise RuntimeError(f"reference failed rc={rc}: {lib.ref_last_error().decode(errors='replace')[:300]}")
    return out


def rounding_for(path: str) -> int:
    """The int8 rounding rule of the reference code path that is the checker of record for a case."""
    return ROUND_ADD_HALF_TRUNC if path.startswith("packed") or path == "port_packed_epilogue" else ROUND_HALF_AWAY


def nchw_to_nhwc_padded(a: np.ndarray, cpad: int) -> np.ndarray:
    n, c, h, w = a.shape
    out = np.zeros((n, h, w, cpad), dtype=a.dtype)
    out[..., :c] = a.transpose(0, 2, 3, 1)
    return out


def nhwc_padded_to_nchw(a: np.ndarray, c: int) -> np.ndarray:
    return np.ascontiguousarray(a[..., :c].transpose(0, 3, 1, 2))
