"""ctypes binding of include/otter_b200.h (one Python function per exported symbol, plus two small
convenience classes used by the tests and the benchmark)."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

F32_NCHW, S8_NHWC, S32_NHWC = 0, 1, 2
ROUND_ADD_HALF_TRUNC, ROUND_HALF_AWAY = 0, 1
ACT_NONE, ACT_RELU, ACT_LRELU, ACT_RELU6 = 0, 1, 2, 3
KERNEL_DEPTHWISE, KERNEL_DENSE_UMMA, KERNEL_DENSE_DIRECT = 1, 2, 3

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libotter_b200.so"


class OtterB200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"otter_b200 error {code}: {what}")
        self.code = code


class OttConvDesc(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("cin", "cout", "kh", "kw", "sh", "sw", "ph", "pw", "dh", "dw", "groups", "bias_term",
                                       "int8_scale_term", "act_type")] + [("act_param0", C.c_float), ("rounding", C.c_int)]


# name -> (restype, argtypes); the single list of what include/otter_b200.h declares
vp, i32, u64p, sz = C.c_void_p, C.c_int, C.POINTER(C.c_uint64), C.c_size_t
SIGNATURES = {
    "ott_cuda_device_count": (i32, [C.POINTER(i32)]),
    "ott_ctx_create": (i32, [i32, C.POINTER(vp)]),
    "ott_ctx_destroy": (i32, [vp]),
    "ott_last_error": (C.c_char_p, [vp]),
    "ott_ctx_stream": (vp, [vp]),
    "ott_sync": (i32, [vp]),
    "ott_set_wait_limit_ms": (i32, [vp, i32]),
    "ott_debug_wait_probe": (i32, [vp]),
    "ott_debug_mma_rate": (i32, [vp, i32, i32, i32, i32, i32, C.POINTER(C.c_float)]),
    "ott_set_depthwise_tensor_cores": (i32, [vp, i32]),
    "ott_debug_fail_alloc_after": (i32, [vp, i32]),
    "ott_debug_guard_bands": (i32, [vp, C.c_size_t]),
    "ott_debug_check_guards": (i32, [vp, C.POINTER(C.c_long)]),
    "ott_malloc": (i32, [vp, sz, C.POINTER(vp)]),
    "ott_free": (i32, [vp, vp]),
    "ott_alloc_stats": (i32, [vp, u64p, u64p, u64p, u64p]),
    "ott_alloc_release_cached": (i32, [vp]),
    "ott_host_alloc": (i32, [sz, C.POINTER(vp)]),
    "ott_host_free": (i32, [vp]),
    "ott_memcpy_h2d": (i32, [vp, vp, vp, sz]),
    "ott_memcpy_d2h": (i32, [vp, vp, vp, sz]),
    "ott_memset": (i32, [vp, vp, i32, sz]),
    "ott_memcpy_overlapped": (i32, [vp, i32, vp, vp, sz]),
    "ott_event_create": (i32, [vp, C.POINTER(vp)]),
    "ott_event_record": (i32, [vp, vp]),
    "ott_event_elapsed_ms": (i32, [vp, vp, C.POINTER(C.c_float)]),
    "ott_event_destroy": (i32, [vp]),
    "ott_nhwc_channels": (i32, [i32]),
    "ott_quantize_f32_nchw_to_s8_nhwc": (i32, [vp, vp, i32, i32, i32, i32, vp, i32, i32, vp]),
    "ott_conv_int8_create": (i32, [vp, C.POINTER(OttConvDesc), vp, vp, vp, vp, i32, vp, i32, C.POINTER(vp)]),
    "ott_conv_int8_destroy": (i32, [vp, vp]),
    "ott_conv_int8_kernel_kind": (i32, [vp]),
    "ott_conv_int8_kernel_name": (C.c_char_p, [vp, vp, i32, i32, i32, i32]),
    "ott_conv_int8_out_shape": (i32, [vp, i32, i32, C.POINTER(i32), C.POINTER(i32)]),
    "ott_conv_int8_forward": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, i32, vp]),
    "ott_conv_int8_forward_ex": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, i32, vp]),
    "ott_conv_int8_forward_gather": (i32, [vp, vp, vp, vp, i32, vp, i32, i32, i32, vp, i32, vp]),
    "ott_conv_int8_create_gathered": (i32, [vp, C.POINTER(OttConvDesc), vp, vp, vp, vp, i32, vp, i32, i32, vp, vp, vp, C.POINTER(vp)]),
    "ott_conv_int8_gathered_layout": (i32, [vp, C.POINTER(i32), vp, i32]),
    "ott_conv_int8_set_f32_plane_map": (i32, [vp, vp, vp, i32]),
    "ott_conv_int8_forward_io": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "ott_unit_int8_create": (i32, [vp, vp, vp, vp, C.POINTER(vp)]),
    "ott_unit_int8_forward_io": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "ott_unit_int8_destroy": (i32, [vp, vp]),
    "ott_dwpw_int8_create": (i32, [vp, vp, vp, C.POINTER(vp)]),
    "ott_dwpw_int8_forward_io": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "ott_dwpw_int8_destroy": (i32, [vp, vp]),
    "ott_gather_channels_f32": (i32, [vp, vp, vp, i32, vp, i32, i32, i32, vp]),
    "ott_add_gather_f32": (i32, [vp, vp, vp, i32, vp, vp, vp, i32, vp, i32, i32, i32, vp]),
    "ott_conv_int8_forward_maxpool": (i32, [vp, vp, vp, i32, i32, i32, i32, vp]),
    "ott_conv_int8_forward_maxpool_s8": (i32, [vp, vp, vp, i32, i32, i32, i32, vp]),
    "ott_conv_int8_forward_host": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, i32]),
    "ott_conv_int8_forward_noalloc": (i32, [vp, vp, vp, i32, i32, i32, vp, i32]),
    "ott_conv_f32_create": (i32, [vp, C.POINTER(OttConvDesc), vp, vp, C.POINTER(vp)]),
    "ott_conv_f32_forward": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "ott_conv_f32_destroy": (i32, [vp, vp]),
    "ott_launch_count": (C.c_uint64, [vp]),
    "ott_copy_channels_f32": (i32, [vp, vp, i32, i32, i32, vp, i32, i32, i32, i32, i32, i32]),
    "ott_maxpool_f32_nchw": (i32, [vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]),
    "ott_upsample_bilinear_f32_nchw": (i32, [vp, vp, i32, i32, i32, i32, i32, i32, C.c_double, C.c_double, i32, vp]),
    "ott_upsample_nearest_f32_nchw": (i32, [vp, vp, i32, i32, i32, i32, i32, i32, C.c_double, C.c_double, i32, vp]),
    "ott_add_f32": (i32, [vp, vp, vp, vp, sz]),
    "ott_graph_capture_begin": (i32, [vp]),
    "ott_graph_capture_end": (i32, [vp, C.POINTER(vp)]),
    "ott_graph_seal": (i32, [vp, vp]),
    "ott_graph_launch": (i32, [vp, vp]),
    "ott_graph_destroy": (i32, [vp, vp]),
    "ott_nanodet_detect": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, C.c_float, C.c_float, vp, vp, i32]),
    "ott_activation_f32": (i32, [vp, vp, sz, i32, C.c_float]),
    # include/otter_b200_net.h
    "ott_net_create": (i32, [i32, C.POINTER(vp)]),
    "ott_net_destroy": (i32, [vp]),
    "ott_net_last_error": (C.c_char_p, [vp]),
    "ott_net_context": (vp, [vp]),
    "ott_net_set_option": (i32, [vp, C.c_char_p, i32]),
    "ott_net_add_layer": (i32, [vp, C.c_char_p]),
    "ott_net_compile": (i32, [vp]),
    "ott_net_load_otter": (i32, [vp, C.c_char_p]),
    "ott_net_load_model": (i32, [vp, C.c_char_p, C.c_char_p, i32]),
    "ott_otter_parse_text": (i32, [C.c_char_p, C.c_char_p, i32]),
    "ott_net_layer_count": (i32, [vp]),
    "ott_net_layer_info": (i32, [vp, i32, C.c_char_p, i32, C.c_char_p, i32, C.POINTER(i32)]),
    "ott_net_blob_shape": (i32, [vp, C.c_char_p, C.POINTER(i32)]),
    "ott_net_blob_element_size": (i32, [vp, C.c_char_p]),
    "ott_net_group_create": (i32, [C.POINTER(i32), i32, C.POINTER(vp)]),
    "ott_net_group_destroy": (i32, [vp]),
    "ott_net_group_size": (i32, [vp]),
    "ott_net_group_member": (vp, [vp, i32]),
    "ott_net_group_last_error": (C.c_char_p, [vp]),
    "ott_net_group_partition": (None, [i32, i32, i32, C.POINTER(i32), C.POINTER(i32)]),
    "ott_net_group_forward": (i32, [vp, C.c_char_p, vp, i32, i32, i32, i32, i32, C.POINTER(C.c_char_p), C.POINTER(vp)]),
    "ott_net_layer_routing": (i32, [vp, i32, C.POINTER(i32)]),
    "ott_net_set_conv_params": (i32, [vp, C.c_char_p, vp, vp, vp, vp, i32, vp, i32]),
    "ott_net_set_conv_params_f32": (i32, [vp, C.c_char_p, vp, vp]),
    "ott_net_capture": (i32, [vp, C.c_char_p, vp, i32, i32, i32, i32, i32, C.POINTER(C.c_char_p), C.POINTER(vp)]),
    "ott_net_graph_launch": (i32, [vp]),
    "ott_net_graph_output": (i32, [vp, i32, C.POINTER(vp), C.POINTER(i32)]),
    "ott_net_graph_destroy": (i32, [vp]),
    "ott_net_forward_rows": (i32, [vp, C.c_char_p, vp, i32, i32, i32, i32, i32, C.c_char_p, vp, i32, C.POINTER(i32), C.POINTER(i32)]),
    "ott_net_profile": (i32, [vp, C.c_char_p, vp, i32, i32, i32, i32, i32, C.c_char_p, C.POINTER(C.c_float)]),
    "ott_net_forward": (i32, [vp, C.c_char_p, vp, i32, i32, i32, i32, i32, i32, C.POINTER(C.c_char_p), C.POINTER(vp)]),
}



class OttConvIO(C.Structure):
    """ott_conv_io of include/otter_b200.h"""
    _fields_ = [("in_dev", C.c_void_p), ("in_dtype", C.c_int), ("sources", C.POINTER(C.c_void_p)), ("n_sources", C.c_int),
                ("out_dev", C.c_void_p), ("out_dtype", C.c_int), ("out_f32_dev", C.c_void_p), ("f32_channel_mask", C.c_void_p),
                ("chunk_dst", C.POINTER(C.c_void_p)), ("chunk_pitch", C.c_void_p), ("n_chunks", C.c_int)]


_lib = None


def library_path() -> Path:
    return _LIB_PATH


def library():
    """Load the native library. Raises if it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise OtterB200Error(-1, f"{_LIB_PATH} is missing; build it with `python -m tensor_b200.build`")
        lib = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def nhwc_channels(c: int) -> int:
    return (c + 15) & ~15


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Context:
    """One GPU: stream + caching allocator (ott_ctx)."""

    def __init__(self, device: int = 0):
        self.lib = library()
        h = C.c_void_p()
        rc = self.lib.ott_ctx_create(device, C.byref(h))
        if rc != 0:
            raise OtterB200Error(rc, f"ott_ctx_create(device={device}) failed (no sm_100 GPU?)")
        self.h = h
        self.device = device

    def check(self, rc: int):
        if rc != 0:
            raise OtterB200Error(rc, self.lib.ott_last_error(self.h).decode(errors="replace"))

    def check_guards(self):
        """With guard bands on (OTT_DEBUG_GUARD_BYTES, ott_debug_guard_bands): raises if a kernel wrote outside a device block."""
        bad = C.c_long(0)
        self.check(self.lib.ott_debug_check_guards(self.h, C.byref(bad)))

    def close(self):
        if self.h:
            h, self.h = self.h, None
            try:
                if os.environ.get("OTT_DEBUG_GUARD_BYTES"):
                    bad = C.c_long(0)
                    rc = self.lib.ott_debug_check_guards(h, C.byref(bad))
                    if rc != 0:
                        raise OtterB200Error(rc, self.lib.ott_last_error(h).decode(errors="replace"))
            finally:
                self.lib.ott_ctx_destroy(h)

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def malloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self.lib.ott_malloc(self.h, nbytes, C.byref(p)))
        return p.value

    def free(self, p: int):
        self.check(self.lib.ott_free(self.h, C.c_void_p(p)))

    def to_device(self, a: np.ndarray) -> int:
        a = np.ascontiguousarray(a)
        p = self.malloc(max(a.nbytes, 1))
        self.check(self.lib.ott_memcpy_h2d(self.h, C.c_void_p(p), _np_ptr(a), a.nbytes))
        self.sync()  # the source is pageable numpy memory
        return p

    def to_host(self, p: int, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        self.check(self.lib.ott_memcpy_d2h(self.h, _np_ptr(out), C.c_void_p(p), out.nbytes))
        self.sync()
        return out

    def memset(self, p: int, value: int, nbytes: int):
        self.check(self.lib.ott_memset(self.h, C.c_void_p(p), value, nbytes))

    def sync(self):
        self.check(self.lib.ott_sync(self.h))

    def alloc_stats(self):
        v = [C.c_uint64() for _ in range(4)]
        self.check(self.lib.ott_alloc_stats(self.h, *[C.byref(x) for x in v]))
        return {"device_mallocs": v[0].value, "cache_hits": v[1].value, "bytes_in_use": v[2].value, "bytes_cached": v[3].value}

    def launch_count(self) -> int:
        return int(self.lib.ott_launch_count(self.h))

    def event(self):
        e = C.c_void_p()
        self.check(self.lib.ott_event_create(self.h, C.byref(e)))
        return e

    def record(self, e):
        self.check(self.lib.ott_event_record(self.h, e))

    def elapsed_ms(self, a, b) -> float:
        ms = C.c_float()
        self.check(self.lib.ott_event_elapsed_ms(a, b, C.byref(ms)))
        return float(ms.value)

    def quantize(self, x_dev: int, n, c, h, w, scales: np.ndarray, rounding: int, out_dev: int):
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        self.check(self.lib.ott_quantize_f32_nchw_to_s8_nhwc(self.h, C.c_void_p(x_dev), n, c, h, w, _np_ptr(scales), scales.size,
                                                              rounding, C.c_void_p(out_dev)))


class ConvInt8:
    """A quantized ConvolutionLayer on the GPU (ott_conv). Array arguments are host numpy arrays in the
    reference's field layouts (weight OIHW int8, bias/scales fp32)."""

    def __init__(self, ctx: Context, *, cin, cout, kh, kw, sh=1, sw=1, ph=0, pw=0, dh=1, dw=1, groups=1, bias_term=1,
                 int8_scale_term=2, act_type=0, act_param0=0.0, rounding=0, weight, bias, w_scales, in_scales, out_scales=None,
                 gathered=None):
        """gathered: None, or (source_channels, channel_source, channel_index) for a layer whose input channels live in
        several int8 NHWC tensors (ott_conv_int8_create_gathered)."""
        self.ctx = ctx
        self.desc = OttConvDesc(cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, bias_term, int8_scale_term, act_type,
                                act_param0, rounding)
        weight = np.ascontiguousarray(weight, dtype=np.int8)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        w_scales = np.ascontiguousarray(w_scales, dtype=np.float32)
        in_scales = np.ascontiguousarray(in_scales, dtype=np.float32)
        out_scales = None if out_scales is None else np.ascontiguousarray(out_scales, dtype=np.float32)
        h = C.c_void_p()
        if gathered is None:
            ctx.check(ctx.lib.ott_conv_int8_create(ctx.h, C.byref(self.desc), _np_ptr(weight), _np_ptr(bias), _np_ptr(w_scales),
                                                   _np_ptr(in_scales), in_scales.size, _np_ptr(out_scales),
                                                   0 if out_scales is None else out_scales.size, C.byref(h)))
        else:
            sc, cs, ci = (np.ascontiguousarray(a, dtype=np.int32) for a in gathered)
            ctx.check(ctx.lib.ott_conv_int8_create_gathered(ctx.h, C.byref(self.desc), _np_ptr(weight), _np_ptr(bias), _np_ptr(w_scales),
                                                            _np_ptr(in_scales), in_scales.size, _np_ptr(out_scales),
                                                            0 if out_scales is None else out_scales.size, sc.size, _np_ptr(sc),
                                                            _np_ptr(cs), _np_ptr(ci), C.byref(h)))
        self.h = h

    @property
    def kernel_kind(self) -> int:
        return self.ctx.lib.ott_conv_int8_kernel_kind(self.h)

    def out_hw(self, h, w):
        oh, ow = C.c_int(), C.c_int()
        self.ctx.check(self.ctx.lib.ott_conv_int8_out_shape(self.h, h, w, C.byref(oh), C.byref(ow)))
        return oh.value, ow.value

    def forward(self, in_dev: int, in_dtype: int, n, h, w, out_dev: int, out_dtype: int, status_dev=None):
        self.ctx.check(self.ctx.lib.ott_conv_int8_forward(self.ctx.h, self.h, C.c_void_p(in_dev), in_dtype, n, h, w,
                                                          C.c_void_p(out_dev), out_dtype, C.c_void_p(status_dev) if status_dev else None))

    def gathered_layout(self):
        """(stored channels, position of every logical channel) of a depthwise layer with gathered input; (0, []) otherwise."""
        stored = C.c_int()
        pos = np.zeros(self.desc.cout, np.int32)
        self.ctx.check(self.ctx.lib.ott_conv_int8_gathered_layout(self.h, C.byref(stored), _np_ptr(pos), pos.size))
        return stored.value, pos

    def set_f32_plane_map(self, plane_of_channel, planes_total: int):
        m = np.ascontiguousarray(plane_of_channel, dtype=np.int32)
        self.ctx.check(self.ctx.lib.ott_conv_int8_set_f32_plane_map(self.ctx.h, self.h, _np_ptr(m), planes_total))

    def forward_io(self, n, h, w, out_dev: int, out_dtype: int, *, in_dev: int = 0, in_dtype: int = S8_NHWC, sources=None,
                   out_f32_dev: int = 0, f32_channels=None, chunk_dst=None, chunk_pitch=None):
        """ott_conv_int8_forward_io: `sources` = device pointers of a gathered layer's int8 inputs; `f32_channels` = output
        channels that are also stored as fp32 planes of out_f32_dev."""
        io = OttConvIO()
        io.in_dev, io.in_dtype = (in_dev or None), in_dtype
        keep = []
        if sources is not None:
            arr = (C.c_void_p * len(sources))(*[C.c_void_p(p) for p in sources])
            keep.append(arr)
            io.sources, io.n_sources = C.cast(arr, C.POINTER(C.c_void_p)), len(sources)
        io.out_dev, io.out_dtype = out_dev, out_dtype
        if out_f32_dev:
            mask = np.zeros((self.desc.cout + 31) // 32, np.uint32)
            for c in f32_channels:
                mask[c >> 5] |= np.uint32(1 << (c & 31))
            keep.append(mask)
            io.out_f32_dev, io.f32_channel_mask = out_f32_dev, mask.ctypes.data
        if chunk_dst is not None:
            arr = (C.c_void_p * len(chunk_dst))(*[C.c_void_p(p) if p else None for p in chunk_dst])
            pitch = np.ascontiguousarray(chunk_pitch, dtype=np.uint32)
            keep += [arr, pitch]
            io.chunk_dst, io.chunk_pitch, io.n_chunks = C.cast(arr, C.POINTER(C.c_void_p)), pitch.ctypes.data, len(chunk_dst)
        self.ctx.check(self.ctx.lib.ott_conv_int8_forward_io(self.ctx.h, self.h, C.byref(io), n, h, w, None))

    def out_array(self, n, h, w, out_dtype):
        oh, ow = self.out_hw(h, w)
        cout = self.desc.cout
        if out_dtype == F32_NCHW:
            return np.empty((n, cout, oh, ow), np.float32)
        if out_dtype == S8_NHWC:
            return np.empty((n, oh, ow, nhwc_channels(cout)), np.int8)
        return np.empty((n, oh, ow, nhwc_channels(cout)), np.int32)

    def forward_host(self, x: np.ndarray, in_dtype: int, out_dtype: int) -> np.ndarray:
        x = np.ascontiguousarray(x)
        if in_dtype == F32_NCHW:
            n, _, h, w = x.shape
        else:
            n, h, w, _ = x.shape
        out = self.out_array(n, h, w, out_dtype)
        self.ctx.check(self.ctx.lib.ott_conv_int8_forward_host(self.ctx.h, self.h, _np_ptr(x), in_dtype, n, h, w, _np_ptr(out), out_dtype))
        return out

    def close(self):
        if self.h:
            self.ctx.lib.ott_conv_int8_destroy(self.ctx.h, self.h)
            self.h = None


class DwPwInt8:
    """A depthwise 3x3 layer and the 1x1 layer behind it as one launch (ott_dwpw). Both layers must outlive the pair."""

    def __init__(self, ctx: Context, dw: "ConvInt8", pw: "ConvInt8"):
        self.ctx, self.cout = ctx, pw.desc.cout
        h = C.c_void_p()
        ctx.check(ctx.lib.ott_dwpw_int8_create(ctx.h, dw.h, pw.h, C.byref(h)))
        self.h = h

    def forward_io(self, n, h, w, out_dev: int, out_dtype: int, *, in_dev: int = 0, sources=None, out_f32_dev: int = 0, f32_channels=None):
        io = OttConvIO()
        io.in_dev, io.in_dtype = (in_dev or None), S8_NHWC
        keep = []
        if sources is not None:
            arr = (C.c_void_p * len(sources))(*[C.c_void_p(p) for p in sources])
            keep.append(arr)
            io.sources, io.n_sources = C.cast(arr, C.POINTER(C.c_void_p)), len(sources)
        io.out_dev, io.out_dtype = out_dev, out_dtype
        if out_f32_dev:
            mask = np.zeros((self.cout + 31) // 32, np.uint32)
            for c in f32_channels:
                mask[c >> 5] |= np.uint32(1 << (c & 31))
            keep.append(mask)
            io.out_f32_dev, io.f32_channel_mask = out_f32_dev, mask.ctypes.data
        self.ctx.check(self.ctx.lib.ott_dwpw_int8_forward_io(self.ctx.h, self.h, C.byref(io), n, h, w, None))

    def close(self):
        if self.h:
            self.ctx.lib.ott_dwpw_int8_destroy(self.ctx.h, self.h)
            self.h = None


class UnitInt8:
    """The chain pw1 -> depthwise 3x3 -> pw2 of three ConvInt8 layers as one launch (ott_unit). pw2 must outlive the unit."""

    def __init__(self, ctx: Context, pw1: "ConvInt8", dw: "ConvInt8", pw2: "ConvInt8"):
        self.ctx, self.cout = ctx, pw2.desc.cout
        h = C.c_void_p()
        ctx.check(ctx.lib.ott_unit_int8_create(ctx.h, pw1.h, dw.h, pw2.h, C.byref(h)))
        self.h = h

    def forward_io(self, n, h, w, out_dev: int, out_dtype: int, *, in_dev: int = 0, sources=None, out_f32_dev: int = 0, f32_channels=None):
        io = OttConvIO()
        io.in_dev, io.in_dtype = (in_dev or None), S8_NHWC
        keep = []
        if sources is not None:
            arr = (C.c_void_p * len(sources))(*[C.c_void_p(p) for p in sources])
            keep.append(arr)
            io.sources, io.n_sources = C.cast(arr, C.POINTER(C.c_void_p)), len(sources)
        io.out_dev, io.out_dtype = out_dev, out_dtype
        if out_f32_dev:
            mask = np.zeros((self.cout + 31) // 32, np.uint32)
            for c in f32_channels:
                mask[c >> 5] |= np.uint32(1 << (c & 31))
            keep.append(mask)
            io.out_f32_dev, io.f32_channel_mask = out_f32_dev, mask.ctypes.data
        self.ctx.check(self.ctx.lib.ott_unit_int8_forward_io(self.ctx.h, self.h, C.byref(io), n, h, w, None))

    def close(self):
        if self.h:
            self.ctx.lib.ott_unit_int8_destroy(self.ctx.h, self.h)
            self.h = None


class ConvF32:
    """An fp32 ConvolutionLayer (int8_scale_term == 0) on the GPU (ott_conv_f32); weight fp32 OIHW, host arrays."""

    def __init__(self, ctx: Context, *, cin, cout, kh, kw, sh=1, sw=1, ph=0, pw=0, dh=1, dw=1, groups=1, act_type=0, act_param0=0.0, weight, bias=None):
        self.ctx = ctx
        self.desc = OttConvDesc(cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, 0 if bias is None else 1, 0, act_type, act_param0, 0)
        weight = np.ascontiguousarray(weight, dtype=np.float32)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        h = C.c_void_p()
        ctx.check(ctx.lib.ott_conv_f32_create(ctx.h, C.byref(self.desc), _np_ptr(weight), _np_ptr(bias), C.byref(h)))
        self.h = h

    def forward_host(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        n, _, h, w = x.shape
        d = self.desc
        oh = (h + 2 * d.ph - d.dh * (d.kh - 1) - 1) // d.sh + 1
        ow = (w + 2 * d.pw - d.dw * (d.kw - 1) - 1) // d.sw + 1
        xd = self.ctx.to_device(x)
        od = self.ctx.malloc(n * d.cout * oh * ow * 4)
        try:
            self.ctx.check(self.ctx.lib.ott_conv_f32_forward(self.ctx.h, self.h, C.c_void_p(xd), n, h, w, C.c_void_p(od)))
            return self.ctx.to_host(od, (n, d.cout, oh, ow), np.float32)
        finally:
            self.ctx.free(xd)
            self.ctx.free(od)

    def close(self):
        if self.h:
            self.ctx.lib.ott_conv_f32_destroy(self.ctx.h, self.h)
            self.h = None


class NetGraph:
    """A captured forward (ott_net_capture): launch() replays it on the Net's stream."""

    def __init__(self, net, handle, n_out):
        self.net, self.h, self.n_out = net, handle, n_out

    def launch(self):
        self.net.check(self.net.lib.ott_net_graph_launch(self.h))

    def output(self, index: int):
        """(device pointer, shape) of output `index`."""
        p = C.c_void_p()
        shape = (C.c_int * 4)()
        self.net.check(self.net.lib.ott_net_graph_output(self.h, index, C.byref(p), shape))
        return p.value, tuple(shape)

    def close(self):
        if self.h:
            self.net.lib.ott_net_graph_destroy(self.h)
            self.h = None


def parse_otter_text(text: str):
    """The library's .otter reader on a string: list of option dictionaries (values as strings), in file order."""
    lib = library()
    cap = 64 + 4 * len(text)
    buf = C.create_string_buffer(cap)
    n = lib.ott_otter_parse_text(text.encode(), buf, cap)
    if n < 0:
        raise OtterB200Error(n, "otter syntax error")
    out = []
    for line in buf.value.decode().splitlines():
        out.append(dict(item.split("=", 1) for item in line.split(";")))
    return out


class Net:
    """ctypes wrapper over include/otter_b200_net.h: a Net built from the reference's LayerOption key/value pairs."""

    def __init__(self, device: int = 0, handle=None):
        self.lib = library()
        self.owned = handle is None
        if handle is None:
            handle = C.c_void_p()
            rc = self.lib.ott_net_create(device, C.byref(handle))
            if rc != 0:
                raise OtterB200Error(rc, "ott_net_create failed")
        self.h = handle
        self.layers = []

    def check(self, rc: int):
        if rc != 0:
            raise OtterB200Error(rc, self.lib.ott_net_last_error(self.h).decode(errors="replace"))

    def set_option(self, key: str, value: int):
        """A field of Net::option (lightmode, int8_rounding, fuse_first_layer_pool, int8_handover, ...); before compile()."""
        self.check(self.lib.ott_net_set_option(self.h, key.encode(), int(value)))

    def add_layer(self, **options):
        """options as in the .otter format, e.g. type="Convolution", name="conv1", input="data", out_channels=24, ..."""
        self.layers.append(dict(options))
        text = ";".join(f"{k}={v}" for k, v in options.items())
        self.check(self.lib.ott_net_add_layer(self.h, text.encode()))

    def compile(self):
        self.check(self.lib.ott_net_compile(self.h))

    def load_otter(self, path: str):
        """Read a .otter text graph (the reference's model-structure format) and compile it."""
        self.check(self.lib.ott_net_load_otter(self.h, str(path).encode()))

    def load_model(self, otter_path: str, weight_path: str, weight_type: str = "ncnn"):
        """Graph from a .otter file, parameters from a weight file ("ncnn": the .bin of a quantized ncnn model)."""
        self.check(self.lib.ott_net_load_model(self.h, str(otter_path).encode(), str(weight_path).encode(), 1 if weight_type == "ncnn" else 0))

    def context(self) -> "Context":
        ctx = Context.__new__(Context)
        ctx.lib, ctx.h, ctx.device = self.lib, C.c_void_p(self.lib.ott_net_context(self.h)), None
        return ctx

    def layer_infos(self):
        out = []
        for i in range(self.lib.ott_net_layer_count(self.h)):
            t, n = C.create_string_buffer(64), C.create_string_buffer(128)
            g = (C.c_int * 12)()
            self.check(self.lib.ott_net_layer_info(self.h, i, t, 64, n, 128, g))
            keys = ("cin", "cout", "kh", "kw", "sh", "sw", "ph", "pw", "groups", "bias_term", "int8_scale_term", "act_type")
            r = (C.c_int * 3)()
            self.check(self.lib.ott_net_layer_routing(self.h, i, r))
            out.append({"type": t.value.decode(), "name": n.value.decode(), **dict(zip(keys, list(g))),
                        "gathered_sources": r[0], "out_int8_channels": r[1], "out_f32_channels": r[2]})
        return out

    def blob_shape(self, name: str):
        s = (C.c_int * 4)()
        self.check(self.lib.ott_net_blob_shape(self.h, name.encode(), s))
        return tuple(s)

    def set_conv_params(self, layer: str, weight, bias, w_scales, in_scales, out_scales=None):
        weight = np.ascontiguousarray(weight, dtype=np.int8)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        w_scales = np.ascontiguousarray(w_scales, dtype=np.float32)
        in_scales = np.ascontiguousarray(in_scales, dtype=np.float32)
        out_scales = None if out_scales is None else np.ascontiguousarray(out_scales, dtype=np.float32)
        self.check(self.lib.ott_net_set_conv_params(self.h, layer.encode(), _np_ptr(weight), _np_ptr(bias), _np_ptr(w_scales),
                                                    _np_ptr(in_scales), in_scales.size, _np_ptr(out_scales),
                                                    0 if out_scales is None else out_scales.size))

    def set_conv_params_f32(self, layer: str, weight, bias=None):
        weight = np.ascontiguousarray(weight, dtype=np.float32)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.check(self.lib.ott_net_set_conv_params_f32(self.h, layer.encode(), _np_ptr(weight), _np_ptr(bias)))

    def forward_raw(self, input_blob: str, in_ptr, in_on_device: bool, shape, out_blobs, out_ptrs=None):
        n, c, h, w = shape
        names = (C.c_char_p * len(out_blobs))(*[b.encode() for b in out_blobs])
        ptrs = None
        if out_ptrs is not None:
            ptrs = (C.c_void_p * len(out_blobs))(*out_ptrs)
        self.check(self.lib.ott_net_forward(self.h, input_blob.encode(), in_ptr, 1 if in_on_device else 0, n, c, h, w, len(out_blobs),
                                            names, ptrs))

    def profile(self, input_blob: str, in_ptr, in_on_device: bool, shape, out_blob: str):
        """Per-layer device time in ms (layers serialised by events): [(type, name, ms)]."""
        n, c, h, w = shape
        infos = self.layer_infos()
        ms = (C.c_float * len(infos))()
        self.check(self.lib.ott_net_profile(self.h, input_blob.encode(), in_ptr, 1 if in_on_device else 0, n, c, h, w, out_blob.encode(), ms))
        return [(i["type"], i["name"], float(m)) for i, m in zip(infos, ms)]

    def forward(self, input_blob: str, x: np.ndarray, out_blobs, dtypes=None):
        """Host fp32 NCHW in, list of host arrays out: fp32 NCHW, or int8 NCHW for the blob of a requantizing layer
        (int8_scale_term > 100); dtypes overrides the per-blob choice."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        outs = []
        for i, b in enumerate(out_blobs):
            dt = dtypes[i] if dtypes else (np.int8 if self.lib.ott_net_blob_element_size(self.h, b.encode()) == 1 else np.float32)
            outs.append(np.empty(self.blob_shape(b)[:0] + (x.shape[0],) + self.blob_shape(b)[1:], dtype=dt))
        self.forward_raw(input_blob, _np_ptr(x), False, x.shape, out_blobs, [o.ctypes.data for o in outs])
        return outs

    def capture(self, input_blob: str, in_dev_ptr, shape, out_blobs):
        """Freeze one forward (device input at in_dev_ptr, device outputs) into a CUDA graph; returns a NetGraph."""
        n, c, h, w = shape
        names = (C.c_char_p * len(out_blobs))(*[b.encode() for b in out_blobs])
        g = C.c_void_p()
        self.check(self.lib.ott_net_capture(self.h, input_blob.encode(), in_dev_ptr, n, c, h, w, len(out_blobs), names, C.byref(g)))
        return NetGraph(self, g, len(out_blobs))

    def forward_rows(self, input_blob: str, x: np.ndarray, out_blob: str, capacity_rows: int = 4096):
        """Host fp32 NCHW in, a 2-D blob of data-dependent length out (the detection layer's [count, 6])."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros((capacity_rows, 8), np.float32)
        rows, cols = C.c_int(), C.c_int()
        n, c, h, w = x.shape
        self.check(self.lib.ott_net_forward_rows(self.h, input_blob.encode(), _np_ptr(x), 0, n, c, h, w, out_blob.encode(), _np_ptr(out),
                                                 capacity_rows * 8 // 6, C.byref(rows), C.byref(cols)))
        k = min(rows.value, capacity_rows * 8 // max(cols.value, 1))
        return out.reshape(-1)[:k * cols.value].reshape(k, cols.value).copy(), rows.value

    def close(self):
        if self.h and self.owned:
            h, self.h = self.h, None
            try:
                if os.environ.get("OTT_DEBUG_GUARD_BYTES"):
                    ctx = self.lib.ott_net_context(h)
                    bad = C.c_long(0)
                    rc = self.lib.ott_debug_check_guards(C.c_void_p(ctx), C.byref(bad)) if ctx else 0
                    if rc != 0:
                        raise OtterB200Error(rc, self.lib.ott_last_error(C.c_void_p(ctx)).decode(errors="replace"))
            finally:
                self.lib.ott_net_destroy(h)
        self.h = None


def partition(n: int, parts: int, index: int):
    """(first image, image count) of slice `index` when n images are cut into `parts` contiguous slices (ott_net_group_partition)."""
    first, count = C.c_int(), C.c_int()
    library().ott_net_group_partition(n, parts, index, C.byref(first), C.byref(count))
    return first.value, count.value


class NetGroup:
    """One Net replica per listed device behind one forward call (ott_net_group_*). `members` are Net wrappers over the
    replicas: configure each the same way (add_layer / compile / set_conv_params or load_model)."""

    def __init__(self, devices):
        self.lib = library()
        arr = (C.c_int * len(devices))(*devices)
        h = C.c_void_p()
        rc = self.lib.ott_net_group_create(arr, len(devices), C.byref(h))
        if rc != 0:
            raise OtterB200Error(rc, "ott_net_group_create failed")
        self.h = h
        self.members = [Net(handle=C.c_void_p(self.lib.ott_net_group_member(h, i))) for i in range(len(devices))]

    def forward_raw(self, input_blob: str, in_ptr, shape, out_blobs, out_ptrs):
        n, c, h, w = shape
        names = (C.c_char_p * len(out_blobs))(*[b.encode() for b in out_blobs])
        ptrs = (C.c_void_p * len(out_blobs))(*out_ptrs)
        rc = self.lib.ott_net_group_forward(self.h, input_blob.encode(), in_ptr, n, c, h, w, len(out_blobs), names, ptrs)
        if rc != 0:
            raise OtterB200Error(rc, self.lib.ott_net_group_last_error(self.h).decode(errors="replace"))

    def forward(self, input_blob: str, x: np.ndarray, out_blobs):
        x = np.ascontiguousarray(x, dtype=np.float32)
        m = self.members[0]
        outs = [np.empty((x.shape[0],) + m.blob_shape(b)[1:], dtype=np.int8 if self.lib.ott_net_blob_element_size(m.h, b.encode()) == 1 else np.float32)
                for b in out_blobs]
        self.forward_raw(input_blob, _np_ptr(x), x.shape, out_blobs, [o.ctypes.data for o in outs])
        return outs

    def close(self):
        if self.h:
            for m in self.members:
                m.h = None
            self.lib.ott_net_group_destroy(self.h)
            self.h = None
